// Routing of a mixture-of-experts feed-forward, all on the device (nothing comes back to the host, so a step with a
// routed layer can be captured into a CUDA graph).
//
// llm_route_topk:   s = softmax(z) over all router outputs, or sigmoid(z) of each (float32); the `top` largest of
//                   s + correction (null: of s) are chosen (ties: the lower index), in descending order; the weights are the
//                   chosen s, not renormalised.  A third form compares z + bias itself (the bias where `correction` would be) and
//                   takes the softmax over the chosen outputs alone as weights.  One warp per token.
// llm_moe_plan:     the (token, choice) pairs sorted by expert, stable in the pair's index: source[r] = token of sorted row r,
//                   place[token * top + j] = sorted row of that pair (-1 for a choice >= experts: an expert without tensors),
//                   and the list of row tiles (expert, first row, rows) that llm_gemm_grouped walks, with its count in front.
//                   One block; a warp per expert counts and places by ballots over 32 pairs at a time.
// llm_moe_combine:  out[t] = sum over the token's choices j, in that order, of weight[t, j] * (the expert's output row, or
//                   the token's own input row for an expert without tensors).  The order is fixed: no atomics.
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(128)
route_topk_kernel(const float* __restrict__ z, const float* __restrict__ correction, int* __restrict__ chosen,
                  float* __restrict__ weights, int tokens, int outputs, int top, int sigmoid) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float route_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= tokens) return;
    float* s = route_smem + (size_t)warp * 2 * outputs;      // scores, then choice scores
    float* c = s + outputs;
    const float* row = z + (size_t)t * outputs;
    if (sigmoid == 2) {
        // the outputs themselves (plus a bias, where one is given) are compared; the weights are made after the choice
        for (int i = lane; i < outputs; i += 32) { s[i] = row[i] + (correction ? correction[i] : 0.f); c[i] = s[i]; }
    } else if (sigmoid) {
        for (int i = lane; i < outputs; i += 32) { s[i] = 1.0f / (1.0f + expf(-row[i])); c[i] = s[i] + (correction ? correction[i] : 0.f); }
    } else {
        float m = -INFINITY;
        for (int i = lane; i < outputs; i += 32) m = fmaxf(m, row[i]);
        m = warp_max(m);
        float sum = 0.f;
        for (int i = lane; i < outputs; i += 32) { const float e = expf(row[i] - m); s[i] = e; sum += e; }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int i = lane; i < outputs; i += 32) { s[i] *= inv; c[i] = s[i] + (correction ? correction[i] : 0.f); }
    }
    __syncwarp();
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int i = lane; i < outputs; i += 32)
            if (c[i] > best) { best = c[i]; at = i; }       // strided walk upwards: the lowest index of a lane's ties stays
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (lane == 0) {
            chosen[(size_t)t * top + j] = at;
            weights[(size_t)t * top + j] = s[at];
            c[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (sigmoid == 2 && lane == 0) {
        // softmax over the chosen outputs alone; the first choice is the largest
        float* w = weights + (size_t)t * top;
        const float m = w[0];
        float sum = 0.f;
        for (int j = 0; j < top; ++j) { w[j] = expf(w[j] - m); sum += w[j]; }
        const float inv = 1.0f / sum;
        for (int j = 0; j < top; ++j) w[j] *= inv;
    }
}

__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ chosen, int pairs, int top, int experts, int tile_rows, int* __restrict__ source,
                int* __restrict__ place, int* __restrict__ tiles, int max_tiles, int* __restrict__ counts_out,
                const float* __restrict__ weights, float* __restrict__ row_weight) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ int plan_smem[];          // counts [experts], first rows [experts]
    int* count = plan_smem;
    int* first = plan_smem + experts;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    for (int e = warp; e < experts; e += nwarp) {
        int n = 0;
        for (int i0 = 0; i0 < pairs; i0 += 32) {
            const int i = i0 + lane;
            n += __popc(__ballot_sync(0xffffffffu, i < pairs && chosen[i] == e));
        }
        if (lane == 0) count[e] = n;
    }
    for (int i = threadIdx.x; i < pairs; i += blockDim.x)
        if (chosen[i] >= experts || chosen[i] < 0) place[i] = -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0, n_tiles = 0;
        for (int e = 0; e < experts; ++e) {
            first[e] = row;
            if (counts_out) counts_out[e] = count[e];
            for (int r = 0; r < count[e]; r += tile_rows) {
                if (n_tiles < max_tiles) {
                    int* rec = tiles + 4 + 4 * n_tiles;
                    rec[0] = e; rec[1] = row + r; rec[2] = min(tile_rows, count[e] - r); rec[3] = 0;
                }
                ++n_tiles;
            }
            row += count[e];
        }
        tiles[0] = min(n_tiles, max_tiles); tiles[1] = row; tiles[2] = 0; tiles[3] = 0;
    }
    __syncthreads();
    for (int e = warp; e < experts; e += nwarp) {
        int at = first[e];
        for (int i0 = 0; i0 < pairs; i0 += 32) {
            const int i = i0 + lane;
            const bool mine = i < pairs && chosen[i] == e;
            const unsigned ballot = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int r = at + __popc(ballot & ((1u << lane) - 1u));
                source[r] = i / top;
                place[i] = r;
            }
            at += __popc(ballot);
        }
    }
    if (!row_weight) return;                // the same for the whole block
    __syncthreads();                        // the places above were written by this block
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {     // the pair's weight beside its sorted row
        const int r = place[i];
        if (r >= 0) row_weight[r] = weights[i];
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ place, const int* __restrict__ chosen,
                   const float* __restrict__ weights, const T* __restrict__ x, T* __restrict__ out, int width, int top, int experts) {
    pdl_trigger();
    pdl_wait();
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top; ++j) {
            const int e = chosen[t * top + j];
            const float w = weights ? weights[t * top + j] : 1.0f;
            const float v = e >= experts ? to_f32(x[t * width + c]) : to_f32(y[(size_t)place[t * top + j] * width + c]);
            acc = fmaf(w, v, acc);
        }
        out[t * width + c] = from_f32<T>(acc);
    }
}

// dst[r] = src[index[r]] for r < rows[0] (the count lives on the device), 16 bytes a thread and step when the rows allow it
template <typename T>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const T* __restrict__ src, const int* __restrict__ index, const int* __restrict__ live_rows, T* __restrict__ dst,
                   int width, int vec, const float* __restrict__ row_weight) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    if (r >= live_rows[0]) return;
    const T* from = src + (size_t)index[r] * width;
    T* to = dst + (size_t)r * width;
    if (row_weight) {
        const float w = row_weight[r];
        for (int i = threadIdx.x; i < width; i += blockDim.x) to[i] = from_f32<T>(to_f32(from[i]) * w);
    } else if (vec) {
        const int n = width * (int)sizeof(T) / 16;
        for (int i = threadIdx.x; i < n; i += blockDim.x) reinterpret_cast<uint4*>(to)[i] = reinterpret_cast<const uint4*>(from)[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) to[i] = from[i];
    }
}

}  // namespace

// dst [max_rows, width] <- src rows by index, for the first live_rows[0] rows (a device count, e.g. tiles + 1 of llm_moe_plan).
// row_weight: null, or a factor per gathered row.
LLM_API int llm_gather_rows(const void* src, const int* index, const int* live_rows, void* dst, int dtype, int max_rows, int width,
                            const float* row_weight, cudaStream_t stream) {
    if (max_rows == 0) return 0;
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        const int vec = !((width * sizeof(T)) % 16) && !((uintptr_t)src & 15) && !((uintptr_t)dst & 15);
        llm_launch(gather_rows_kernel<T>, (unsigned)max_rows, 256, 0, stream, (const T*)src, index, live_rows, (T*)dst, width, vec,
                   row_weight);
        LLM_CHECK_LAUNCH("gather_rows");
        return 0;
    });
}

LLM_API int llm_route_topk(const float* z, const float* correction, int* chosen, float* weights, int tokens, int outputs, int top,
                           int sigmoid, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (top < 1 || top > outputs) LLM_FAIL(-1, "route_topk: %d of %d outputs", top, outputs);
    if (sigmoid < 0 || sigmoid > 2) LLM_FAIL(-1, "route_topk: form %d is not known (0 softmax, 1 sigmoid, 2 softmax over the chosen)", sigmoid);
    const size_t smem = (size_t)4 * 2 * outputs * sizeof(float);
    if (smem > 48 * 1024) LLM_FAIL(-1, "route_topk: %d router outputs are more than 1536", outputs);
    llm_launch(route_topk_kernel, (unsigned)((tokens + 3) / 4), 128, smem, stream, z, correction, chosen, weights, tokens, outputs, top,
               sigmoid);
    LLM_CHECK_LAUNCH("route_topk");
    return 0;
}

// tiles: int32 [(max_tiles + 1) * 4]: the first four ints are (count, sorted rows, 0, 0), then one record per tile.
// counts: null, or int32 [experts] that receives every expert's row count (for a caller that wants them on the host).
// weights / row_weight: null, or the pairs' weights [pairs] and a place [pairs] for them in the order of the sorted rows.
LLM_API int llm_moe_plan(const int* chosen, int pairs, int top, int experts, int tile_rows, int* source, int* place, int* tiles,
                         int max_tiles, int* counts, const float* weights, float* row_weight, cudaStream_t stream) {
    if (pairs == 0) return 0;
    if (experts <= 0 || experts > 4096) LLM_FAIL(-1, "moe_plan: %d experts (1 to 4096)", experts);
    llm_launch(moe_plan_kernel, 1, 1024, (size_t)2 * experts * sizeof(int), stream, chosen, pairs, top, experts, tile_rows, source,
               place, tiles, max_tiles, counts, weights, row_weight && weights ? row_weight : nullptr);
    LLM_CHECK_LAUNCH("moe_plan");
    return 0;
}

LLM_API int llm_moe_combine(const void* y, const int* place, const int* chosen, const float* weights, const void* x, void* out,
                            int dtype, int tokens, int width, int top, int experts, cudaStream_t stream) {
    if (tokens == 0) return 0;
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(moe_combine_kernel<T>, (unsigned)tokens, 256, 0, stream, (const T*)y, place, chosen, weights, (const T*)x, (T*)out,
                   width, top, experts);
        LLM_CHECK_LAUNCH("moe_combine");
        return 0;
    });
}

LLM_TRACE_EXPORT(moe_route)
