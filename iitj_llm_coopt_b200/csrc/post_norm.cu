// Norms behind the residual sum, the average over depth, the mean of normed branches and a normed polynomial activation.
// One block per token row, the row held in shared memory as float32, every statistic and sum in float32.
//
// llm_post_norm:    y = (alpha * x + branch) / rms(alpha * x + branch) * gain          (x float32; branch of the engine's type or
//                   float32; gain float32 as it multiplies).  y is written as float32 (`out`), and as the engine's type (`cast`).
//                   With a history [inputs, tokens, width] float32 and weights [inputs]: y is stored as the history's last
//                   entry, and  mixed = sum_j weights[j] * history[j]  (j in order, the new row last) is what `out` and `cast`
//                   receive instead.
// llm_branch_mean:  out = scale * sum_b branch_b / rms(branch_b) * gain_b   for up to four branches, float32 out.
// llm_poly_norm:    act = a z / rms(z) + b z^2 / rms(z^2) + c z^3 / rms(z^3) + e   over a token's row of z, powers element by element.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

template <typename TB, typename TC>
__global__ void __launch_bounds__(kThreads)
post_norm_kernel(const float* x, const TB* __restrict__ branch, float alpha, const float* __restrict__ gain, float eps,
                 float* out, TC* __restrict__ cast, float* history, const float* __restrict__ mix,
                 int inputs, long long entry_stride, int width) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float pn_row[];
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += kThreads) {
        const float v = alpha * x[base + i] + to_f32(branch[base + i]);
        pn_row[i] = v;
        ss += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
    if (!history) {
        for (int i = threadIdx.x; i < width; i += kThreads) {
            const float y = pn_row[i] * inv * gain[i];
            out[base + i] = y;
            if (cast) cast[base + i] = from_f32<TC>(y);
        }
        return;
    }
    // the earlier entries are only read and the last one only written: the reads of four columns run side by side
    const float* __restrict__ earlier = history;
    float* __restrict__ last = history + (size_t)(inputs - 1) * entry_stride;
    const float w_last = mix[inputs - 1];
    for (int i0 = threadIdx.x; i0 < width; i0 += 4 * kThreads) {
        float m[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j + 1 < inputs; ++j) {
            const float wj = mix[j];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = i0 + e * kThreads;
                if (i < width) m[e] = fmaf(wj, earlier[(size_t)j * entry_stride + base + i], m[e]);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = i0 + e * kThreads;
            if (i >= width) continue;
            const float y = pn_row[i] * inv * gain[i];
            last[base + i] = y;
            const float mixed = fmaf(w_last, y, m[e]);
            out[base + i] = mixed;
            if (cast) cast[base + i] = from_f32<TC>(mixed);
        }
    }
}

struct BranchArgs {
    const void* branch[4];
    const float* gain[4];
    int n;
};

template <typename T>
__global__ void __launch_bounds__(kThreads)
branch_mean_kernel(BranchArgs a, float scale, float eps, float* __restrict__ out, int width) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * width;
    float inv[4];
    for (int b = 0; b < a.n; ++b) {
        const T* p = (const T*)a.branch[b] + base;
        float ss = 0.f;
        for (int i = threadIdx.x; i < width; i += kThreads) { const float v = to_f32(p[i]); ss += v * v; }
        inv[b] = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
    }
    for (int i = threadIdx.x; i < width; i += kThreads) {
        float acc = 0.f;
        for (int b = 0; b < a.n; ++b) acc += to_f32(((const T*)a.branch[b])[base + i]) * inv[b] * a.gain[b][i];
        out[base + i] = scale * acc;
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
poly_norm_kernel(const T* __restrict__ z, const float* __restrict__ coef, float eps, T* __restrict__ act, int inner) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * inner;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = threadIdx.x; i < inner; i += kThreads) {
        const float v = to_f32(z[base + i]), v2 = v * v;
        s1 += v2;
        s2 += v2 * v2;
        s3 += v2 * v2 * v2;
    }
    const float n = (float)inner;
    const float r1 = coef[0] / sqrtf(block_sum(s1, red) / n + eps);
    const float r2 = coef[1] / sqrtf(block_sum(s2, red) / n + eps);
    const float r3 = coef[2] / sqrtf(block_sum(s3, red) / n + eps);
    const float e = coef[3];
    for (int i = threadIdx.x; i < inner; i += kThreads) {
        const float v = to_f32(z[base + i]), v2 = v * v;
        act[base + i] = from_f32<T>(r1 * v + r2 * v2 + r3 * v2 * v + e);
    }
}

}  // namespace

// x, out: float32 [tokens, width] (they may be the same); branch [tokens, width] of `branch_dtype`; gain float32 [width]; cast: null or
// [tokens, width] of `cast_dtype`.  history: null, or float32 with `inputs` entries of `entry_stride` numbers each, of which the first
// inputs - 1 are read and the last is written; mix float32 [inputs].
LLM_API int llm_post_norm(const float* x, const void* branch, int branch_dtype, float alpha, const float* gain, float eps, float* out,
                          void* cast, int cast_dtype, float* history, const float* mix, int inputs, long long entry_stride,
                          int tokens, int width, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (width <= 0) LLM_FAIL(-1, "post_norm: width %d", width);
    if (history && (!mix || inputs < 1 || entry_stride < (long long)tokens * width))
        LLM_FAIL(-1, "post_norm: a history needs weights, at least one entry and entries of tokens x width numbers");
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) LLM_FAIL(-1, "post_norm: a row of %d numbers does not fit shared memory", width);
    return llm_dispatch_dtype(branch_dtype, [&](auto tb) {
        using TB = decltype(tb);
        return llm_dispatch_dtype(cast ? cast_dtype : LLM_BF16, [&](auto tc) {
            using TC = decltype(tc);
            if (smem > 48 * 1024) cudaFuncSetAttribute(post_norm_kernel<TB, TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            llm_launch(post_norm_kernel<TB, TC>, (unsigned)tokens, kThreads, smem, stream, x, (const TB*)branch, alpha, gain, eps, out,
                       (TC*)cast, history, mix, inputs, entry_stride, width);
            LLM_CHECK_LAUNCH("post_norm");
            return 0;
        });
    });
}

// branches: `n` pointers (1 to 4) to [tokens, width] of `dtype`; gains: as many pointers to float32 [width].
LLM_API int llm_branch_mean(const void* const* branches, const float* const* gains, int n, int dtype, float scale, float eps, float* out,
                            int tokens, int width, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (n < 1 || n > 4) LLM_FAIL(-1, "branch_mean: %d branches (1 to 4)", n);
    BranchArgs a;
    a.n = n;
    for (int b = 0; b < 4; ++b) { a.branch[b] = b < n ? branches[b] : nullptr; a.gain[b] = b < n ? gains[b] : nullptr; }
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(branch_mean_kernel<T>, (unsigned)tokens, kThreads, 0, stream, a, scale, eps, out, width);
        LLM_CHECK_LAUNCH("branch_mean");
        return 0;
    });
}

// z, act: [tokens, inner] of `dtype`; coef float32 [4]: the factors of the three normed powers and the constant.
LLM_API int llm_poly_norm(const void* z, const float* coef, float eps, void* act, int dtype, int tokens, int inner, cudaStream_t stream) {
    if (tokens == 0 || inner == 0) return 0;
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(poly_norm_kernel<T>, (unsigned)tokens, kThreads, 0, stream, (const T*)z, coef, eps, (T*)act, inner);
        LLM_CHECK_LAUNCH("poly_norm");
        return 0;
    });
}

LLM_TRACE_EXPORT(post_norm)
