// What lies between a grouped attention's fused projection and its attention kernel, for one token per block, with every
// step optional and all arithmetic in float32:
//
//   row = [q: heads x dim | k: kv_heads x dim | v: kv_heads x vdim]   (k and v absent for a layer that reads another layer's
//                                                                    keys and values; v absent when the values are the keys)
//   row += bias                                                      (one float32 number per column of the row)
//   values = the keys as they are at this point                      (`value_from_key`)
//   norm:   1  every head of q and of k divided by its root mean square over dim, times a gain [dim] shared by all heads
//              (null gain: no gain);   2  q as a whole divided by its root mean square over heads x dim, times a gain of that
//              size, and k likewise over kv_heads x dim
//   rotate: the leading rotary_dim numbers of every head of q and k by the token's cos/sin rows (pairs (2i, 2i + 1) when
//           interleaved, else (i, i + rotary_dim / 2))
//   `norm_first` chooses which of the two comes first.
//   q goes back in place (the engine's type); k and the values go into the token's slot of a flat-page cache (key plane
//   [kv_heads, page, dim], then value plane [kv_heads, page, vdim]).
#include "common.cuh"

namespace {

struct QkArgs {
    void* row; int ld;
    const float* bias;
    const float* q_gain; const float* k_gain;
    const float* cos; const float* sin;
    void* cache; const int* slots; long long page_stride; int page_size;
    int heads, kv_heads, dim, vdim, norm, norm_first, rotary_dim, interleaved, own_kv, value_from_key;
    float eps;
};

template <typename T>
__global__ void __launch_bounds__(256)
qk_prepare_kernel(QkArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float qk_smem[];
    __shared__ float red[32];
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const int q_cols = a.heads * a.dim, k_cols = a.own_kv ? a.kv_heads * a.dim : 0;
    const int qk_cols = q_cols + k_cols;
    T* row = (T*)a.row + (size_t)t * a.ld;
    float* x = qk_smem;                                  // q, then k, as float32
    for (int i = threadIdx.x; i < qk_cols; i += blockDim.x) x[i] = to_f32(row[i]) + (a.bias ? a.bias[i] : 0.f);
    __syncthreads();
    const bool store = a.own_kv && a.slots != nullptr;
    const int slot = store ? a.slots[t] : 0;
    T* page = store ? (T*)a.cache + (size_t)(slot / a.page_size) * a.page_stride : nullptr;
    const int off = slot % a.page_size;
    if (store) {
        T* vplane = page + (size_t)a.kv_heads * a.page_size * a.dim;
        const int v_cols = a.kv_heads * a.vdim;
        for (int i = threadIdx.x; i < v_cols; i += blockDim.x) {
            const int g = i / a.vdim, c = i % a.vdim;
            const float v = a.value_from_key ? x[q_cols + i] : to_f32(row[qk_cols + i]) + (a.bias ? a.bias[qk_cols + i] : 0.f);
            vplane[((size_t)g * a.page_size + off) * a.vdim + c] = from_f32<T>(v);
        }
        __syncthreads();                                 // the keys change below
    }
    const int all_heads = a.heads + (a.own_kv ? a.kv_heads : 0);
    const int half = a.rotary_dim / 2;
    const float* cos_t = a.cos ? a.cos + (size_t)t * half : nullptr;
    const float* sin_t = a.sin ? a.sin + (size_t)t * half : nullptr;
    for (int pass = 0; pass < 2; ++pass) {
        const bool do_norm = (pass == 0) == (a.norm_first != 0);
        if (do_norm && a.norm == 1) {
            for (int h = warp; h < all_heads; h += nwarp) {
                float* v = x + (size_t)h * a.dim;
                const float* gain = h < a.heads ? a.q_gain : a.k_gain;
                float ss = 0.f;
                for (int i = lane; i < a.dim; i += 32) ss += v[i] * v[i];
                const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)a.dim + a.eps);
                for (int i = lane; i < a.dim; i += 32) v[i] = v[i] * inv * (gain ? gain[i] : 1.f);
            }
        } else if (do_norm && a.norm == 2) {
            for (int part = 0; part < (a.own_kv ? 2 : 1); ++part) {
                float* v = part ? x + q_cols : x;
                const int n = part ? k_cols : q_cols;
                const float* gain = part ? a.k_gain : a.q_gain;
                float ss = 0.f;
                for (int i = threadIdx.x; i < n; i += blockDim.x) ss += v[i] * v[i];
                const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)n + a.eps);
                for (int i = threadIdx.x; i < n; i += blockDim.x) v[i] = v[i] * inv * (gain ? gain[i] : 1.f);
            }
        } else if (!do_norm && half > 0) {
            for (int i = threadIdx.x; i < all_heads * half; i += blockDim.x) {
                const int h = i / half, p = i % half;
                float* v = x + (size_t)h * a.dim;
                const int ia = a.interleaved ? 2 * p : p, ib = a.interleaved ? 2 * p + 1 : p + half;
                const float u = v[ia], w = v[ib], c = cos_t[p], s = sin_t[p];
                v[ia] = u * c - w * s;
                v[ib] = w * c + u * s;
            }
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < q_cols; i += blockDim.x) row[i] = from_f32<T>(x[i]);
    if (store)
        for (int i = threadIdx.x; i < k_cols; i += blockDim.x) {
            const int g = i / a.dim, c = i % a.dim;
            page[((size_t)g * a.page_size + off) * a.dim + c] = from_f32<T>(x[q_cols + i]);
        }
}

}  // namespace

// row: [tokens, ld] of `dtype`, the fused projection (layout in the file's head).  bias: null or float32 with one number per
// column used.  norm: 0 none, 1 per head (gains [dim] or null), 2 whole projection (gains [heads * dim] and [kv_heads * dim] or
// null).  cos / sin: float32 [tokens, rotary_dim / 2] (rotary_dim 0: no rotation).  slots null: nothing is stored.
LLM_API int llm_qk_prepare(void* row, int ld, const float* bias, const float* q_gain, const float* k_gain, const float* cos,
                           const float* sin, void* cache, const int* slots, long long page_stride, int page_size, int dtype,
                           int tokens, int heads, int kv_heads, int dim, int vdim, int norm, int norm_first, int rotary_dim,
                           int interleaved, int own_kv, int value_from_key, float eps, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (rotary_dim % 2 || rotary_dim < 0 || rotary_dim > dim || (rotary_dim && (!cos || !sin)))
        LLM_FAIL(-1, "qk_prepare: rotary_dim %d must be even, at most dim %d, and come with tables", rotary_dim, dim);
    if (norm < 0 || norm > 2) LLM_FAIL(-1, "qk_prepare: norm form %d is not known", norm);
    if (value_from_key && vdim != dim) LLM_FAIL(-1, "qk_prepare: values that are the keys have the keys' size (%d, %d)", vdim, dim);
    QkArgs a;
    a.row = row; a.ld = ld; a.bias = bias; a.q_gain = q_gain; a.k_gain = k_gain; a.cos = cos; a.sin = sin; a.cache = cache;
    a.slots = slots; a.page_stride = page_stride; a.page_size = page_size; a.heads = heads; a.kv_heads = kv_heads; a.dim = dim;
    a.vdim = vdim; a.norm = norm; a.norm_first = norm_first; a.rotary_dim = rotary_dim; a.interleaved = interleaved;
    a.own_kv = own_kv; a.value_from_key = value_from_key; a.eps = eps;
    const size_t smem = (size_t)(heads + (own_kv ? kv_heads : 0)) * dim * sizeof(float);
    if (smem > 200 * 1024) LLM_FAIL(-1, "qk_prepare: a row of %zu bytes does not fit shared memory", smem);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        if (smem > 48 * 1024) cudaFuncSetAttribute(qk_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        llm_launch(qk_prepare_kernel<T>, (unsigned)tokens, 256, smem, stream, a);
        LLM_CHECK_LAUNCH("qk_prepare");
        return 0;
    });
}

LLM_TRACE_EXPORT(qk_prepare)
