// Norms that sit on a branch's output, and the clamped gated activation.
//
// llm_norm_add:     residual[t] (+)= branch[t] * rsqrt(mean(branch[t]^2) + eps) * weight   (float32 statistics and sum),
//                   and optionally a copy of the new residual row in the engine's type, which the next sub-layer reads.
//                   One block per row, the row held in registers between the two passes, sums in a fixed order.
//                   With a second gain the new residual row is normed as well, into rows of the engine's type: the norm
//                   in front of the next sub-layer of a design that has norms on both sides of its sub-layers.
// llm_rmsnorm_rows: out[t] = in[t] * rsqrt(mean(in[t]^2) + eps) * weight for rows of the engine's type with strides of their
//                   own (some columns of a wider product), float32 statistics.
// llm_glu_clamped:  act = g * sigmoid(slope * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit),
//                   from one [T, 2 * inner] row of gate columns followed by up columns.
// llm_glu_act:      act = f(gate) * up from such a row, f = silu (0) or the tanh form of gelu (1).
#include "common.cuh"

namespace {

constexpr int kNormThreads = 256;
constexpr int kNormPer = 8;          // elements a thread holds: rows up to 2048 * ... are walked in rounds of 2048

template <typename TB, typename TW, typename TC>
__global__ void __launch_bounds__(kNormThreads)
norm_add_kernel(float* __restrict__ residual, const TB* __restrict__ branch, const TW* __restrict__ weight,
                TC* __restrict__ cast, int width, float eps, int accumulate, const TW* __restrict__ next_weight,
                TC* __restrict__ next_out) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const TB* b = branch + row * width;
    float* res = residual + row * width;
    float ss = 0.f;
    float held[kNormPer];
    // first pass: sum of squares (the first kNormPer rounds of the row stay in registers)
#pragma unroll
    for (int j = 0; j < kNormPer; ++j) {
        const int i = threadIdx.x + j * kNormThreads;
        held[j] = i < width ? to_f32(b[i]) : 0.f;
        ss += held[j] * held[j];
    }
    for (int i = threadIdx.x + kNormPer * kNormThreads; i < width; i += kNormThreads) {
        const float v = to_f32(b[i]);
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll
    for (int j = 0; j < kNormPer; ++j) {
        const int i = threadIdx.x + j * kNormThreads;
        if (i < width) {
            float y = held[j] * inv * to_f32(weight[i]);
            if (accumulate) y += res[i];
            res[i] = y;
            held[j] = y;
            if (cast) cast[row * width + i] = from_f32<TC>(y);
        }
    }
    float ss2 = 0.f;
    for (int i = threadIdx.x + kNormPer * kNormThreads; i < width; i += kNormThreads) {
        float y = to_f32(b[i]) * inv * to_f32(weight[i]);
        if (accumulate) y += res[i];
        res[i] = y;
        ss2 += y * y;
        if (cast) cast[row * width + i] = from_f32<TC>(y);
    }
    if (!next_out) return;                 // the same for the whole block
    // the norm of the new row (what was held is zero beyond the row's end)
#pragma unroll
    for (int j = 0; j < kNormPer; ++j) ss2 += held[j] * held[j];
    const float inv2 = 1.0f / sqrtf(block_sum(ss2, red) / (float)width + eps);
#pragma unroll
    for (int j = 0; j < kNormPer; ++j) {
        const int i = threadIdx.x + j * kNormThreads;
        if (i < width) next_out[row * width + i] = from_f32<TC>(held[j] * inv2 * to_f32(next_weight[i]));
    }
    for (int i = threadIdx.x + kNormPer * kNormThreads; i < width; i += kNormThreads)
        next_out[row * width + i] = from_f32<TC>(res[i] * inv2 * to_f32(next_weight[i]));
}

template <typename T>
__global__ void __launch_bounds__(128)
rmsnorm_rows_kernel(const T* __restrict__ in, long long ld_in, T* __restrict__ out, long long ld_out, const float* __restrict__ weight,
                    int width, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const T* x = in + (size_t)blockIdx.x * ld_in;
    T* y = out + (size_t)blockIdx.x * ld_out;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = to_f32(x[i]); ss += v * v; }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) y[i] = from_f32<T>(to_f32(x[i]) * inv * weight[i]);
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void glu_act_kernel(const T* __restrict__ gu, T* __restrict__ act, int tokens, int inner, int kind) {
    pdl_trigger();
    pdl_wait();
    const size_t n = (size_t)tokens * inner;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inner, c = i % inner;
        const float g = to_f32(gu[t * 2 * inner + c]), u = to_f32(gu[t * 2 * inner + inner + c]);
        act[i] = from_f32<T>((kind == 1 ? gelu_tanh_f(g) : g / (1.0f + expf(-g))) * u);
    }
}

template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gu, T* __restrict__ act, int tokens, int inner, float limit, float slope) {
    pdl_trigger();
    pdl_wait();
    const size_t n = (size_t)tokens * inner;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inner, c = i % inner;
        const float g = fminf(to_f32(gu[t * 2 * inner + c]), limit);
        const float u = fminf(fmaxf(to_f32(gu[t * 2 * inner + inner + c]), -limit), limit);
        act[i] = from_f32<T>(g / (1.0f + expf(-slope * g)) * (u + 1.0f));
    }
}

}  // namespace

// branch [tokens, width] of `branch_dtype`; weight float32 or bfloat16 (`weight_dtype`); cast: null or [tokens, width] of
// `cast_dtype`.  accumulate == 0 writes the normed row instead of adding it (an embedding's norm).
LLM_API int llm_norm_add(float* residual, const void* branch, int branch_dtype, const void* weight, int weight_dtype,
                         void* cast, int cast_dtype, int tokens, int width, float eps, int accumulate, const void* next_weight,
                         void* next_out, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (width <= 0) LLM_FAIL(-1, "norm_add: width %d", width);
    if ((next_weight == nullptr) != (next_out == nullptr)) LLM_FAIL(-1, "norm_add: the second norm needs a gain and a place for its rows");
    return llm_dispatch_dtype(branch_dtype, [&](auto tb) {
        using TB = decltype(tb);
        return llm_dispatch_dtype(weight_dtype, [&](auto tw) {
            using TW = decltype(tw);
            return llm_dispatch_dtype(cast || next_out ? cast_dtype : LLM_BF16, [&](auto tc) {
                using TC = decltype(tc);
                llm_launch(norm_add_kernel<TB, TW, TC>, (unsigned)tokens, kNormThreads, 0, stream, residual, (const TB*)branch,
                           (const TW*)weight, (TC*)cast, width, eps, accumulate, (const TW*)next_weight, (TC*)next_out);
                LLM_CHECK_LAUNCH("norm_add");
                return 0;
            });
        });
    });
}

// in / out: rows of `dtype` with strides ld_in / ld_out (in elements); weight float32 [width].
LLM_API int llm_rmsnorm_rows(const void* in, long long ld_in, void* out, long long ld_out, const float* weight, int dtype, int tokens,
                             int width, float eps, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (width <= 0) LLM_FAIL(-1, "rmsnorm_rows: width %d", width);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(rmsnorm_rows_kernel<T>, (unsigned)tokens, 128, 0, stream, (const T*)in, ld_in, (T*)out, ld_out, weight, width, eps);
        LLM_CHECK_LAUNCH("rmsnorm_rows");
        return 0;
    });
}

// kind: 0 silu, 1 the tanh form of gelu.
LLM_API int llm_glu_act(const void* gu, void* act, int dtype, int tokens, int inner, int kind, cudaStream_t stream) {
    if (tokens == 0 || inner == 0) return 0;
    if (kind != 0 && kind != 1) LLM_FAIL(-1, "glu_act: activation code %d is not known", kind);
    const size_t n = (size_t)tokens * inner;
    const unsigned blocks = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(glu_act_kernel<T>, blocks, 256, 0, stream, (const T*)gu, (T*)act, tokens, inner, kind);
        LLM_CHECK_LAUNCH("glu_act");
        return 0;
    });
}

LLM_API int llm_glu_clamped(const void* gu, void* act, int dtype, int tokens, int inner, float limit, float slope,
                            cudaStream_t stream) {
    if (tokens == 0 || inner == 0) return 0;
    const size_t n = (size_t)tokens * inner;
    const unsigned blocks = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(glu_clamped_kernel<T>, blocks, 256, 0, stream, (const T*)gu, (T*)act, tokens, inner, limit, slope);
        LLM_CHECK_LAUNCH("glu_clamped");
        return 0;
    });
}

LLM_TRACE_EXPORT(branch_norm)
