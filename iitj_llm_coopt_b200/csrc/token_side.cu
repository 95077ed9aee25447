// A layer's own input from the token itself: every token has a second embedding row, of which each layer reads its slice.
//
// llm_token_side_gate:  out[t, d] = gelu_tanh(gate[t, d]) * table[ids[t], offset + d]   for d < dim, where gate [T, dim] was
//                       projected from the stream and table [vocab, table_width] holds the slices of all layers side by side.
//                       The tanh form of gelu, in float32.
#include "common.cuh"

namespace {

template <typename T>
__global__ void token_side_gate_kernel(const T* __restrict__ gate, const T* __restrict__ table, const int* __restrict__ ids,
                                       T* __restrict__ out, int tokens, int dim, int table_width, int offset) {
    pdl_trigger();
    pdl_wait();
    const size_t n = (size_t)tokens * dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / dim, d = i % dim;
        const float z = to_f32(gate[i]);
        const float g = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        out[i] = from_f32<T>(g * to_f32(table[(size_t)ids[t] * table_width + offset + d]));
    }
}

}  // namespace

LLM_API int llm_token_side_gate(const void* gate, const void* table, const int* ids, void* out, int dtype, int tokens, int dim,
                                int table_width, int offset, cudaStream_t stream) {
    if (tokens == 0 || dim == 0) return 0;
    if (offset < 0 || offset + dim > table_width)
        LLM_FAIL(-1, "token_side_gate: columns [%d, %d) lie outside rows of %d", offset, offset + dim, table_width);
    const size_t n = (size_t)tokens * dim;
    const unsigned blocks = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(token_side_gate_kernel<T>, blocks, 256, 0, stream, (const T*)gate, (const T*)table, ids, (T*)out, tokens, dim,
                   table_width, offset);
        LLM_CHECK_LAUNCH("token_side_gate");
        return 0;
    });
}

LLM_TRACE_EXPORT(token_side)
