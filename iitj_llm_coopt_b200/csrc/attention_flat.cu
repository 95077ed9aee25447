// Attention over caches whose pages are flat rows: the key plane [kv_heads, page, key_dim] followed by the value plane
// [kv_heads, page, value_dim], or the key plane alone when the values are the leading value_dim numbers of the key rows
// (one latent row per token that every query head scores against and sums up).  Key and value sizes are independent and
// need not be multiples of anything; float32 or bfloat16 storage, float32 arithmetic.
//
// llm_latent_prepare:  per token, from the fused projection row [heads x (dim + rot_dim) | kv_rank | rot_dim]:
//                      latent = rmsnorm(row[kv_rank part]) * gain, shared key part rotated, both stored as one cache row;
//                      every head's rotated query part written behind the place of its absorbed part in q_out.
// llm_headnorm_store:  per token, every query head and key head divided by its root mean square and multiplied by a
//                      gain vector shared by all heads (optional); queries in place, keys and values into the cache.
// llm_attention_flat:  softmax(score) over the keys [max(0, p - window + 1), p] (window 0: from 0), times the values,
//                      optionally times sigmoid(gate) (one gate number per head, or one per output number).  The score of
//                      query position p and key position j is  s = scale * temp(p) * q . k,  then  s = cap * tanh(s / cap)
//                      (cap > 0),  then  s -= slope[head] * (p - j)  (slopes given), with the query temperature
//                      temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1)  (every > 0).  With `sinks` every row's denominator
//                      also holds exp(sink[head]), a term without key or value that is neither scaled nor masked.  One warp per (token, head); keys are
//                      walked in tiles of 32 that start at multiples of 32 of the key position, so a row's sums run in an
//                      order that depends on its own position alone.
#include "common.cuh"

namespace {

constexpr int kWarps = 4;

// cos / sin of pair p of token t; pairs are (2p, 2p + 1) when interleaved, else (p, p + half)
template <typename TI, typename TO>
__device__ __forceinline__ void rotate_row(const TI* __restrict__ in, TO* __restrict__ out, int n, int rotary_dim, int interleaved,
                                           const float* __restrict__ cos_t, const float* __restrict__ sin_t, int first, int step) {
    const int half = rotary_dim / 2;
    for (int p = first; p < half; p += step) {
        const int a = interleaved ? 2 * p : p, b = interleaved ? 2 * p + 1 : p + half;
        const float x = to_f32(in[a]), y = to_f32(in[b]), c = cos_t[p], s = sin_t[p];
        out[a] = from_f32<TO>(x * c - y * s);
        out[b] = from_f32<TO>(y * c + x * s);
    }
    for (int i = rotary_dim + first; i < n; i += step) out[i] = from_f32<TO>(to_f32(in[i]));
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ qd, int ld, const T* __restrict__ kv, int ld_kv, const float* __restrict__ cos,
                      const float* __restrict__ sin, int rotary_dim,
                      int interleaved, const float* __restrict__ gain, float eps, T* __restrict__ q_out, T* __restrict__ cache,
                      const int* __restrict__ slots, long long page_stride, int page_size, int heads, int dim, int rot_dim, int rank) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int t = blockIdx.x;
    const T* row = qd + (size_t)t * ld;
    const T* low = kv + (size_t)t * ld_kv;             // [rank latent numbers | rot_dim numbers of the shared key part]
    const int out_row = rank + rot_dim;
    const float* cos_t = cos ? cos + (size_t)t * (rotary_dim / 2) : nullptr;
    const float* sin_t = sin ? sin + (size_t)t * (rotary_dim / 2) : nullptr;
    // every head's rotated query part
    for (int h = 0; h < heads; ++h)
        rotate_row(row + h * (dim + rot_dim) + dim, q_out + (size_t)t * heads * out_row + (size_t)h * out_row + rank, rot_dim,
                   rotary_dim, interleaved, cos_t, sin_t, threadIdx.x, blockDim.x);
    // the latent row's statistics (all threads take part, whether the row is stored or not)
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_f32(low[i]);
        ss += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)rank + eps);
    if (!slots) return;
    const int slot = slots[t];
    T* dst = cache + (size_t)(slot / page_size) * page_stride + (size_t)(slot % page_size) * out_row;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<T>(to_f32(low[i]) * inv * gain[i]);
    rotate_row(low + rank, dst + rank, rot_dim, rotary_dim, interleaved, cos_t, sin_t, threadIdx.x, blockDim.x);
}

template <typename T>
__global__ void __launch_bounds__(128)
headnorm_store_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                      T* __restrict__ cache, const int* __restrict__ slots, long long page_stride, int page_size, int heads,
                      int kv_heads, int dim, int vdim) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    T* row = qkv + (size_t)t * ld;
    const int slot = slots ? slots[t] : 0;
    T* page = slots ? cache + (size_t)(slot / page_size) * page_stride : nullptr;
    const int off = slot % page_size;
    for (int h = warp; h < heads + kv_heads; h += nwarp) {
        T* v = row + (size_t)h * dim;
        const bool is_key = h >= heads;
        if (is_key && !page) continue;
        const float* gain = is_key ? k_gain : q_gain;
        float inv = 1.f;
        if (gain) {
            float ss = 0.f;
            for (int i = lane; i < dim; i += 32) { const float x = to_f32(v[i]); ss += x * x; }
            inv = 1.0f / sqrtf(warp_sum(ss) / (float)dim + eps);
        }
        T* dst = is_key ? page + ((size_t)(h - heads) * page_size + off) * dim : v;
        if (is_key || gain)
            for (int i = lane; i < dim; i += 32) dst[i] = from_f32<T>(gain ? to_f32(v[i]) * inv * gain[i] : to_f32(v[i]));
    }
    if (!page) return;
    const T* vals = row + (size_t)(heads + kv_heads) * dim;
    T* vplane = page + (size_t)kv_heads * page_size * dim;
    for (int i = threadIdx.x; i < kv_heads * vdim; i += blockDim.x) {
        const int g = i / vdim, c = i % vdim;
        vplane[((size_t)g * page_size + off) * vdim + c] = vals[i];
    }
}

template <typename T> __device__ __forceinline__ float dot_any(const T* __restrict__ k, const float* __restrict__ q, int d, bool vec);

template <> __device__ __forceinline__ float dot_any<float>(const float* __restrict__ k, const float* __restrict__ q, int d, bool vec) {
    float acc = 0.f;
    int i = 0;
    if (vec)
        for (; i + 4 <= d; i += 4) {
            const float4 kv = *reinterpret_cast<const float4*>(k + i);
            acc = fmaf(kv.x, q[i], acc); acc = fmaf(kv.y, q[i + 1], acc);
            acc = fmaf(kv.z, q[i + 2], acc); acc = fmaf(kv.w, q[i + 3], acc);
        }
    for (; i < d; ++i) acc = fmaf(k[i], q[i], acc);
    return acc;
}

template <> __device__ __forceinline__ float dot_any<__nv_bfloat16>(const __nv_bfloat16* __restrict__ k, const float* __restrict__ q,
                                                                    int d, bool vec) {
    float acc = 0.f;
    int i = 0;
    if (vec)
        for (; i + 8 <= d; i += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(k + i);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(p[j]);
                acc = fmaf(f.x, q[i + 2 * j], acc);
                acc = fmaf(f.y, q[i + 2 * j + 1], acc);
            }
        }
    for (; i < d; ++i) acc = fmaf(__bfloat162float(k[i]), q[i], acc);
    return acc;
}

template <typename T, int OWN>
__global__ void __launch_bounds__(kWarps * 32)
attention_flat_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ cache, long long page_stride,
                      const int* __restrict__ block_table, int table_width, const int* __restrict__ token_request,
                      const int* __restrict__ positions, const float* __restrict__ gate, int gate_cols, T* __restrict__ out,
                      int out_stride, int tokens, int heads, int kv_heads, int key_dim, int value_dim, int shared_value,
                      int page_size, int window, float scale, float softcap, const float* __restrict__ slopes, float temp_coef,
                      int temp_every, const float* __restrict__ sinks, int vec) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float q_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * kWarps + warp;
    if (item >= (long long)tokens * heads) return;  // whole warp leaves together
    const int t = (int)(item / heads), h = (int)(item % heads);
    const int hk = h / (heads / kv_heads);
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (size_t)token_request[t] * table_width;
    if (temp_every > 0) scale *= 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f);
    const float slope = slopes ? slopes[h] : 0.f;
    const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;

    float* qs = q_smem + (size_t)warp * ((key_dim + 3) & ~3);
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * key_dim;
    for (int i = lane; i < key_dim; i += 32) qs[i] = to_f32(qrow[i]);
    __syncwarp();

    const size_t key_head = (size_t)hk * page_size * key_dim;
    // where a key's value row lies relative to the key row
    const size_t value_plane = (size_t)kv_heads * page_size * key_dim + (size_t)hk * page_size * value_dim;
    float acc[OWN];
#pragma unroll
    for (int i = 0; i < OWN; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int k0 = lo & ~31; k0 <= pos; k0 += 32) {
        const int j = k0 + lane;
        const bool valid = j >= lo && j <= pos;
        long long koff = 0, voff = 0;
        float s = -INFINITY;
        if (valid) {
            const size_t page = (size_t)table[j / page_size] * page_stride;
            const int o = j % page_size;
            koff = (long long)(page + key_head + (size_t)o * key_dim);
            voff = shared_value ? koff : (long long)(page + value_plane + (size_t)o * value_dim);
            s = scale * dot_any<T>(cache + koff, qs, key_dim, vec != 0);
            if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
            s -= slope * (float)(pos - j);
        }
        const float m_new = fmaxf(m, warp_max(s));   // finite: every tile holds a visible key
        const float corr = expf(m - m_new);          // 0 on the first tile (m = -inf)
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < OWN; ++i) acc[i] *= corr;
        for (int jj = 0; jj < 32; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long vo = __shfl_sync(0xffffffffu, voff, jj);
            if (pj == 0.f) continue;  // same for the whole warp
            const T* vrow = cache + vo;
#pragma unroll
            for (int i = 0; i < OWN; ++i) {
                const int d = lane + 32 * i;
                if (d < value_dim) acc[i] = fmaf(pj, to_f32(vrow[d]), acc[i]);
            }
        }
        m = m_new;
    }
    T* orow = out + (size_t)t * out_stride + (size_t)h * value_dim;
    if (sinks) l += expf(sinks[h] - m);      // a term without a key or a value, once in the row's denominator
    float inv = 1.0f / l;
    if (gate && gate_cols == 1) inv *= 1.0f / (1.0f + expf(-gate[(size_t)t * heads + h]));
    const float* grow = gate && gate_cols > 1 ? gate + ((size_t)t * heads + h) * value_dim : nullptr;
#pragma unroll
    for (int i = 0; i < OWN; ++i) {
        const int d = lane + 32 * i;
        if (d < value_dim) orow[d] = from_f32<T>(grow ? acc[i] * inv / (1.0f + expf(-grow[d])) : acc[i] * inv);
    }
}

}  // namespace

// qd: rows of heads x (dim + rot_dim) query numbers (stride ld); kv: rows of rank + rot_dim numbers (stride ld_kv), which may
// be columns of the same product as qd or of another one.
LLM_API int llm_latent_prepare(const void* qd, int ld, const void* kv, int ld_kv, const float* cos, const float* sin,
                               int rotary_dim, int interleaved,
                               const float* gain, float eps, void* q_out, void* cache, const int* slots, long long page_stride,
                               int page_size, int dtype, int tokens, int heads, int dim, int rot_dim, int rank, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (rotary_dim % 2 || rotary_dim > rot_dim || (rotary_dim && (!cos || !sin)))
        LLM_FAIL(-1, "latent_prepare: rotary_dim %d must be even, at most rot_dim %d, and come with tables", rotary_dim, rot_dim);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(latent_prepare_kernel<T>, (unsigned)tokens, 128, 0, stream, (const T*)qd, ld, (const T*)kv, ld_kv, cos, sin,
                   rotary_dim, interleaved, gain, eps, (T*)q_out, (T*)cache, slots, page_stride, page_size, heads, dim, rot_dim, rank);
        LLM_CHECK_LAUNCH("latent_prepare");
        return 0;
    });
}

LLM_API int llm_headnorm_store(void* qkv, int ld, const float* q_gain, const float* k_gain, float eps, void* cache,
                               const int* slots, long long page_stride, int page_size, int dtype, int tokens, int heads,
                               int kv_heads, int dim, int vdim, cudaStream_t stream) {
    if (tokens == 0) return 0;
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(headnorm_store_kernel<T>, (unsigned)tokens, 128, 0, stream, (T*)qkv, ld, q_gain, k_gain, eps, (T*)cache, slots,
                   page_stride, page_size, heads, kv_heads, dim, vdim);
        LLM_CHECK_LAUNCH("headnorm_store");
        return 0;
    });
}

LLM_API int llm_attention_flat(const void* q, int q_stride, const void* cache, long long page_stride, const int* block_table,
                               int table_width, const int* token_request, const int* positions, const float* gate, int gate_cols,
                               void* out, int out_stride, int dtype, int tokens, int heads, int kv_heads, int key_dim, int value_dim,
                               int shared_value, int page_size, int window, float scale, float softcap, const float* slopes,
                               float temp_coef, int temp_every, const float* sinks, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (kv_heads <= 0 || heads % kv_heads) LLM_FAIL(-1, "attention_flat: heads %d is not a multiple of kv_heads %d", heads, kv_heads);
    if (value_dim <= 0 || value_dim > 512 || key_dim <= 0 || key_dim > 2048)
        LLM_FAIL(-1, "attention_flat: value_dim %d must be in [1, 512], key_dim %d in [1, 2048]", value_dim, key_dim);
    if (shared_value && value_dim > key_dim) LLM_FAIL(-1, "attention_flat: shared values are a part of the key rows");
    if (gate && gate_cols != 1 && gate_cols != value_dim)
        LLM_FAIL(-1, "attention_flat: a gate has one number per head or one per output number (%d, value_dim %d)", gate_cols, value_dim);
    const long long items = (long long)tokens * heads;
    const long long blocks = (items + kWarps - 1) / kWarps;
    if (blocks > 0x7fffffffLL) LLM_FAIL(-1, "attention_flat: too many (token, head) pairs: %lld", items);
    const size_t smem = (size_t)kWarps * ((key_dim + 3) & ~3) * sizeof(float);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        const int per = 16 / (int)sizeof(T);          // elements of a 16-byte load
        const int vec = !(key_dim % per) && !(page_stride % per) && !((uintptr_t)cache & 15);
#define LLM_FLAT_CASE(OWN)                                                                                                  \
        llm_launch(attention_flat_kernel<T, OWN>, (unsigned)blocks, kWarps * 32, smem, stream, (const T*)q, q_stride,       \
                   (const T*)cache, page_stride, block_table, table_width, token_request, positions, gate, gate_cols, (T*)out,     \
                   out_stride, tokens, heads, kv_heads, key_dim, value_dim, shared_value, page_size, window, scale, softcap,    \
                   slopes, temp_coef, temp_every, sinks, vec)
        if (value_dim <= 64) LLM_FLAT_CASE(2);
        else if (value_dim <= 128) LLM_FLAT_CASE(4);
        else if (value_dim <= 256) LLM_FLAT_CASE(8);
        else LLM_FLAT_CASE(16);
#undef LLM_FLAT_CASE
        LLM_CHECK_LAUNCH("attention_flat");
        return 0;
    });
}

LLM_TRACE_EXPORT(attention_flat)
