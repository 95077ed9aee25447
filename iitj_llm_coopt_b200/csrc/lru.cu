// A gated linear recurrence per channel (Griffin's recurrent unit with real gates), with its short causal convolution:
//
//   z_t = zx_t + bias_x                               (zx: the input branch's projection, columns [x_col, x_col + width) of `proj`)
//   u_t = conv_bias + sum_j taps[:, j] z_(t - n + 1 + j)        n taps, the last is the current token's; zeros before a request's
//                                                     first token; a request's last n - 1 rows of z are part of its state
//   r_t = sigmoid(Ra u_t + ra_bias),  i_t = sigmoid(Ri u_t + ri_bias)     Ra, Ri block-diagonal: `blocks` square matrices [out, in]
//   a_t = exp(-c r_t softplus(lam)),  S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t       S float32, zero for a new request
//   out_t = S_t * gelu_tanh(zy_t + bias_y)            (zy: the gate branch's projection, columns [y_col, y_col + width))
//
// Everything after the projections is float32; the weights of the gates are read as stored (the engine's type) and widened.
// State per request: [taps, width] float32, row 0 is S, rows 1 .. taps - 1 the last rows of z, oldest first.
//
// llm_lru_conv:   u (float32 [tokens, width]) from proj and the state's rows of z.
// llm_lru_gates:  a and b = sqrt(1 - a^2) i u (float32 [tokens, width]) from u; FMA tiles with a fixed order along k.
// llm_lru_step:   all three at once for a step in which every request brings one token.
// llm_lru_scan:   the recurrence, out, and the new state.  Short portions: one thread per (request, channel) walks the tokens.
//                 Long portions are cut into segments of kSegment tokens: every segment's (product of a, end value from zero)
//                 first, then the segments' starting values one after the other, then every segment again from its start.
#include "common.cuh"

namespace {

constexpr int kSegment = 64;

__device__ __forceinline__ float gelu_tanh_lru(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(256)
lru_conv_kernel(const T* __restrict__ proj, int ld, int x_col, const float* __restrict__ bias_x, const float* __restrict__ taps_w,
                const float* __restrict__ conv_bias, int taps, const float* __restrict__ state, const int* __restrict__ state_slots,
                const int* __restrict__ token_request, const int* __restrict__ cu_seqlens, float* __restrict__ u, int width) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = token_request[t], start = cu_seqlens[b];
    const float* st = state + (size_t)state_slots[b] * taps * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = conv_bias ? conv_bias[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int src = t - (taps - 1) + j;
            // rows before the portion's first token come from the state: row 1 + (taps - 1) + (src - start)
            const float z = src >= start ? to_f32(proj[(size_t)src * ld + x_col + c]) + (bias_x ? bias_x[c] : 0.f)
                                         : st[(size_t)(taps + src - start) * width + c];
            acc = fmaf(taps_w[(size_t)c * taps + j], z, acc);
        }
        u[(size_t)t * width + c] = acc;
    }
}

constexpr int GT = 64, GN = 128, GK = 16;      // tokens x outputs of a block's tile, and the k chunk
constexpr int GPAD = 4;                        // shared rows padded so that the transposing stores spread over the banks

// Eight neighbouring numbers as float32: one 16-byte read of bfloat16, two of float32 (`vec`: the address allows it), else one by one;
// numbers from `n` on read as zero.
__device__ __forceinline__ void load8(const __nv_bfloat16* p, int n, bool vec, float (&v)[8]) {
    if (vec && n >= 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = j < n ? __bfloat162float(p[j]) : 0.f;
    }
}
__device__ __forceinline__ void load8(const float* p, int n, bool vec, float (&v)[8]) {
    if (vec && n >= 8) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = j < n ? p[j] : 0.f;
    }
}

// Eight neighbouring numbers as they are stored (16-byte reads), converted later: what a thread holds of the next k chunk while it
// computes the current one.
template <typename T> struct Raw8;
template <> struct Raw8<__nv_bfloat16> {
    uint4 v;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void get(float (&f)[8]) const {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 x = __bfloat1622float2(h[j]); f[2 * j] = x.x; f[2 * j + 1] = x.y; }
    }
};
template <> struct Raw8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) { a = *reinterpret_cast<const float4*>(p); b = *reinterpret_cast<const float4*>(p + 4); }
    __device__ __forceinline__ void get(float (&f)[8]) const {
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
};

// Both gate products as FMA tiles: a thread holds 8 tokens x 4 outputs of each matrix; operands pass through shared memory with k as
// the slow index, so that a thread's tokens and outputs are neighbours (float4 reads); the sum along k runs in its natural order.
// A thread whose rows and chunk lie wholly inside reads its share of the next chunk into registers before it computes the current one.
template <typename T>
__global__ void __launch_bounds__(256, 2)
lru_gates_kernel(const float* __restrict__ u, const T* __restrict__ ra, const T* __restrict__ ri, const float* __restrict__ ra_bias,
                 const float* __restrict__ ri_bias, const float* __restrict__ lam, float decay_scale, float* __restrict__ a_out,
                 float* __restrict__ b_out, int tokens, int width, int blocks) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) float us[GK][GT + GPAD];
    __shared__ __align__(16) float was[GK][GN + GPAD];
    __shared__ __align__(16) float wis[GK][GN + GPAD];
    const int bs = width / blocks;
    const int col_tiles = (bs + GN - 1) / GN;
    const int blk = blockIdx.y / col_tiles, n0 = (blockIdx.y % col_tiles) * GN;
    const int t0 = blockIdx.x * GT;
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;      // outputs 4 tx .. 4 tx + 3; tokens 8 ty .. 8 ty + 7
    float accr[8][4], acci[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) accr[i][j] = acci[i][j] = 0.f;
    const T* wa = ra + (size_t)blk * bs * bs;
    const T* wi = ri + (size_t)blk * bs * bs;
    const bool wvec = bs % 8 == 0 && !((uintptr_t)ra & 15) && !((uintptr_t)ri & 15);
    const bool uvec = width % 4 == 0 && bs % 4 == 0 && !((uintptr_t)u & 15);
    const int ur = threadIdx.x / 4, ukq = (threadIdx.x % 4) * 4;       // this thread's share of u: four k of one token
    const int wr = threadIdx.x / 2, wkg = (threadIdx.x % 2) * 8;       // and of both matrices: eight k of one output row
    const float* up = u + (size_t)(t0 + ur) * width + blk * bs + ukq;
    const T* wap = wa + (size_t)(n0 + wr) * bs + wkg;
    const T* wip = wi + (size_t)(n0 + wr) * bs + wkg;
    const bool inside = wvec && uvec && t0 + ur < tokens && n0 + wr < bs;
    float4 next_u;
    Raw8<T> next_a, next_i;
    bool have = inside && GK <= bs;
    if (have) { next_u = *reinterpret_cast<const float4*>(up); next_a.load(wap); next_i.load(wip); }
    for (int k0 = 0; k0 < bs; k0 += GK) {
        if (have) {
            float va[8], vi[8];
            next_a.get(va);
            next_i.get(vi);
            us[ukq][ur] = next_u.x; us[ukq + 1][ur] = next_u.y; us[ukq + 2][ur] = next_u.z; us[ukq + 3][ur] = next_u.w;
#pragma unroll
            for (int j = 0; j < 8; ++j) { was[wkg + j][wr] = va[j]; wis[wkg + j][wr] = vi[j]; }
        } else {
            const int uleft = t0 + ur < tokens ? bs - (k0 + ukq) : 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) us[ukq + j][ur] = j < uleft ? up[k0 + j] : 0.f;
            const int wleft = n0 + wr < bs ? bs - (k0 + wkg) : 0;
            float va[8], vi[8];
            load8(wap + k0, wleft, false, va);
            load8(wip + k0, wleft, false, vi);
#pragma unroll
            for (int j = 0; j < 8; ++j) { was[wkg + j][wr] = va[j]; wis[wkg + j][wr] = vi[j]; }
        }
        have = inside && k0 + 2 * GK <= bs;
        if (have) { next_u = *reinterpret_cast<const float4*>(up + k0 + GK); next_a.load(wap + k0 + GK); next_i.load(wip + k0 + GK); }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GK; ++k) {
            const float4 a4 = *reinterpret_cast<const float4*>(&was[k][4 * tx]);
            const float4 i4 = *reinterpret_cast<const float4*>(&wis[k][4 * tx]);
            const float4 u0 = *reinterpret_cast<const float4*>(&us[k][8 * ty]);
            const float4 u1 = *reinterpret_cast<const float4*>(&us[k][8 * ty + 4]);
            const float uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
            const float av[4] = {a4.x, a4.y, a4.z, a4.w}, iv[4] = {i4.x, i4.y, i4.z, i4.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    accr[i][j] = fmaf(uv[i], av[j], accr[i][j]);
                    acci[i][j] = fmaf(uv[i], iv[j], acci[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int t = t0 + 8 * ty + i, n = n0 + 4 * tx + j;
            if (t >= tokens || n >= bs) continue;
            const int c = blk * bs + n;
            const float r = 1.0f / (1.0f + expf(-(accr[i][j] + ra_bias[c])));
            const float g = 1.0f / (1.0f + expf(-(acci[i][j] + ri_bias[c])));
            const float l = lam[c];
            const float sp = l > 20.f ? l : log1pf(expf(l));
            const float a = expf(-decay_scale * r * sp);
            a_out[(size_t)t * width + c] = a;
            b_out[(size_t)t * width + c] = sqrtf(fmaxf(1.0f - a * a, 0.f)) * g * u[(size_t)t * width + c];
        }
}

// The new rows of z of a request's state, for channel c: the last taps - 1 of (old rows, this portion's rows).  Row j is filled in
// rising order from a row behind it (an old row further on, or one of the portion's), so nothing that is still needed is overwritten.
template <typename T>
__device__ __forceinline__ void lru_shift_state(float* st, const T* __restrict__ proj, int ld, int x_col, const float* __restrict__ bias_x,
                                                int taps, int start, int end, int width, int c) {
    const int keep = taps - 1;
    for (int j = 0; j < keep; ++j) {
        const int src = end - keep + j;                 // token row; before `start`: the state's row 1 + keep + (src - start) > 1 + j
        st[(size_t)(1 + j) * width + c] = src >= start ? to_f32(proj[(size_t)src * ld + x_col + c]) + (bias_x ? bias_x[c] : 0.f)
                                                       : st[(size_t)(1 + keep + src - start) * width + c];
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
lru_scan_walk_kernel(const float* __restrict__ a, const float* __restrict__ b, const T* __restrict__ proj, int ld, int y_col, int x_col,
                     const float* __restrict__ bias_y, const float* __restrict__ bias_x, int taps, float* __restrict__ state,
                     const int* __restrict__ state_slots, const int* __restrict__ cu_seqlens, T* __restrict__ out, int width, int write) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (c >= width) return;
    const int start = cu_seqlens[r], end = cu_seqlens[r + 1];
    float* st = state + (size_t)state_slots[r] * taps * width;
    float S = st[c];
    const float by = bias_y ? bias_y[c] : 0.f;
    for (int t = start; t < end; ++t) {
        S = fmaf(a[(size_t)t * width + c], S, b[(size_t)t * width + c]);
        out[(size_t)t * width + c] = from_f32<T>(S * gelu_tanh_lru(to_f32(proj[(size_t)t * ld + y_col + c]) + by));
    }
    if (write && end > start) {
        st[c] = S;
        lru_shift_state(st, proj, ld, x_col, bias_x, taps, start, end, width, c);
    }
}

// A step in which every request brings one token: convolution, gates, recurrence and the new state in one kernel.  One block per
// (request, gate block): it holds the block's u in shared memory, a warp per output row walks k with its lanes (a fixed order), and
// since no other block reads this block's channels of the state, it brings them up to date itself.
template <typename T>
__global__ void __launch_bounds__(1024)
lru_step_kernel(const T* __restrict__ proj, int ld, int y_col, int x_col, const float* __restrict__ bias_y, const float* __restrict__ bias_x,
                const float* __restrict__ taps_w, const float* __restrict__ conv_bias, int taps, const T* __restrict__ ra,
                const T* __restrict__ ri, const float* __restrict__ ra_bias, const float* __restrict__ ri_bias, const float* __restrict__ lam,
                float decay_scale, float* __restrict__ state, const int* __restrict__ state_slots, const int* __restrict__ cu_seqlens,
                T* __restrict__ out, int width, int blocks, int write) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float step_u[];
    const int bs = width / blocks, blk = blockIdx.x, r = blockIdx.y;
    const int t = cu_seqlens[r];
    if (cu_seqlens[r + 1] <= t) return;                    // the request brings nothing: the whole block leaves
    float* st = state + (size_t)state_slots[r] * taps * width;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int c = threadIdx.x; c < bs; c += blockDim.x) {
        const int ch = blk * bs + c;
        const float z = to_f32(proj[(size_t)t * ld + x_col + ch]) + (bias_x ? bias_x[ch] : 0.f);
        float acc = conv_bias ? conv_bias[ch] : 0.f;
        for (int j = 0; j + 1 < taps; ++j) acc = fmaf(taps_w[(size_t)ch * taps + j], st[(size_t)(1 + j) * width + ch], acc);
        step_u[c] = fmaf(taps_w[(size_t)ch * taps + taps - 1], z, acc);
    }
    __syncthreads();
    const T* wa = ra + (size_t)blk * bs * bs;
    const T* wi = ri + (size_t)blk * bs * bs;
    const bool vec = bs % 8 == 0 && !((uintptr_t)ra & 15) && !((uintptr_t)ri & 15);
    const int nwarp = blockDim.x >> 5;
    for (int n0 = warp * 4; n0 < bs; n0 += nwarp * 4) {      // four rows a warp at a time, a lane takes runs of eight k
        // what lane r needs for row n0 + r after the sums is asked for first, so that it arrives while the weights do
        const int n = n0 + lane;
        const bool mine = lane < 4 && n < bs;
        const int ch = blk * bs + (mine ? n : 0);
        const float e_rab = mine ? ra_bias[ch] : 0.f, e_rib = mine ? ri_bias[ch] : 0.f, e_lam = mine ? lam[ch] : 0.f;
        const float e_s = mine ? st[ch] : 0.f;
        const float e_y = mine ? to_f32(proj[(size_t)t * ld + y_col + ch]) + (bias_y ? bias_y[ch] : 0.f) : 0.f;
        float sa[4] = {0.f, 0.f, 0.f, 0.f}, si[4] = {0.f, 0.f, 0.f, 0.f};
        for (int k = lane * 8; k < bs; k += 256) {
            float uv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) uv[j] = k + j < bs ? step_u[k + j] : 0.f;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                if (n0 + r >= bs) continue;
                float va[8], vi[8];
                load8(wa + (size_t)(n0 + r) * bs + k, bs - k, vec, va);
                load8(wi + (size_t)(n0 + r) * bs + k, bs - k, vec, vi);
#pragma unroll
                for (int j = 0; j < 8; ++j) { sa[r] = fmaf(uv[j], va[j], sa[r]); si[r] = fmaf(uv[j], vi[j], si[r]); }
            }
        }
        float ma = 0.f, mi = 0.f;                            // lane r keeps row n0 + r
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float ta = warp_sum(sa[r]), ti = warp_sum(si[r]);
            if (lane == r) { ma = ta; mi = ti; }
        }
        if (mine) {
            const float g = 1.0f / (1.0f + expf(-(ma + e_rab)));
            const float gi = 1.0f / (1.0f + expf(-(mi + e_rib)));
            const float a = expf(-decay_scale * g * (e_lam > 20.f ? e_lam : log1pf(expf(e_lam))));
            const float S = fmaf(a, e_s, sqrtf(fmaxf(1.0f - a * a, 0.f)) * gi * step_u[n]);
            out[(size_t)t * width + ch] = from_f32<T>(S * gelu_tanh_lru(e_y));
            if (write) st[ch] = S;
        }
    }
    if (!write) return;
    for (int c = threadIdx.x; c < bs; c += blockDim.x) {   // every read of these rows lies before the barrier above
        const int ch = blk * bs + c;
        for (int j = 1; j + 1 < taps; ++j) st[(size_t)j * width + ch] = st[(size_t)(j + 1) * width + ch];
        if (taps > 1) st[(size_t)(taps - 1) * width + ch] = to_f32(proj[(size_t)t * ld + x_col + ch]) + (bias_x ? bias_x[ch] : 0.f);
    }
}

// pass 1: every segment's product of a and its end value from zero
__global__ void __launch_bounds__(128)
lru_segment_sums_kernel(const float* __restrict__ a, const float* __restrict__ b, const int* __restrict__ cu_seqlens,
                        float* __restrict__ seg_a, float* __restrict__ seg_b, int width, int segments) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y / segments, s = blockIdx.y % segments;
    if (c >= width) return;
    const int start = cu_seqlens[r] + s * kSegment, end = min(cu_seqlens[r + 1], start + kSegment);
    float A = 1.f, B = 0.f;
    for (int t = start; t < end; ++t) {
        const float at = a[(size_t)t * width + c];
        A *= at;
        B = fmaf(at, B, b[(size_t)t * width + c]);
    }
    seg_a[(size_t)blockIdx.y * width + c] = A;
    seg_b[(size_t)blockIdx.y * width + c] = B;
}

// pass 2: the segments' starting values, one after the other (left in seg_b), the new state
template <typename T>
__global__ void __launch_bounds__(128)
lru_segment_starts_kernel(const float* __restrict__ seg_a, float* __restrict__ seg_b, const T* __restrict__ proj, int ld, int x_col,
                          const float* __restrict__ bias_x, int taps, float* __restrict__ state, const int* __restrict__ state_slots,
                          const int* __restrict__ cu_seqlens, int width, int segments, int write) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (c >= width) return;
    const int start = cu_seqlens[r], end = cu_seqlens[r + 1];
    float* st = state + (size_t)state_slots[r] * taps * width;
    float S = st[c];
    const int used = (end - start + kSegment - 1) / kSegment;
    for (int s = 0; s < used; ++s) {
        const size_t at = ((size_t)r * segments + s) * width + c;
        const float next = fmaf(seg_a[at], S, seg_b[at]);
        seg_b[at] = S;
        S = next;
    }
    if (write && end > start) {
        st[c] = S;
        lru_shift_state(st, proj, ld, x_col, bias_x, taps, start, end, width, c);
    }
}

// pass 3: every segment again, from its starting value
template <typename T>
__global__ void __launch_bounds__(128)
lru_segment_apply_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ seg_start,
                         const T* __restrict__ proj, int ld, int y_col, const float* __restrict__ bias_y,
                         const int* __restrict__ cu_seqlens, T* __restrict__ out, int width, int segments) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y / segments, s = blockIdx.y % segments;
    if (c >= width) return;
    const int start = cu_seqlens[r] + s * kSegment, end = min(cu_seqlens[r + 1], start + kSegment);
    if (start >= end) return;
    float S = seg_start[(size_t)blockIdx.y * width + c];
    const float by = bias_y ? bias_y[c] : 0.f;
    for (int t = start; t < end; ++t) {
        S = fmaf(a[(size_t)t * width + c], S, b[(size_t)t * width + c]);
        out[(size_t)t * width + c] = from_f32<T>(S * gelu_tanh_lru(to_f32(proj[(size_t)t * ld + y_col + c]) + by));
    }
}

}  // namespace

LLM_API int llm_lru_segment() { return kSegment; }

// proj [tokens, ld] of `dtype`; bias_x, conv_bias float32 [width] or null; taps_w float32 [width, taps]; state float32 [slots, taps, width];
// u float32 [tokens, width].
LLM_API int llm_lru_conv(const void* proj, int ld, int x_col, const float* bias_x, const float* taps_w, const float* conv_bias, int taps,
                         const float* state, const int* state_slots, const int* token_request, const int* cu_seqlens, float* u,
                         int dtype, int tokens, int width, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (taps < 1) LLM_FAIL(-1, "lru_conv: %d taps", taps);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(lru_conv_kernel<T>, (unsigned)tokens, 256, 0, stream, (const T*)proj, ld, x_col, bias_x, taps_w, conv_bias, taps, state,
                   state_slots, token_request, cu_seqlens, u, width);
        LLM_CHECK_LAUNCH("lru_conv");
        return 0;
    });
}

// ra, ri [blocks, width / blocks, width / blocks] of `dtype` ([out, in] each); biases and lam float32 [width]; a_out, b_out float32.
LLM_API int llm_lru_gates(const float* u, const void* ra, const void* ri, const float* ra_bias, const float* ri_bias, const float* lam,
                          float decay_scale, float* a_out, float* b_out, int dtype, int tokens, int width, int blocks,
                          cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (blocks < 1 || width % blocks) LLM_FAIL(-1, "lru_gates: width %d is not a multiple of %d blocks", width, blocks);
    const int bs = width / blocks;
    dim3 grid((unsigned)((tokens + GT - 1) / GT), (unsigned)(blocks * ((bs + GN - 1) / GN)));
    if (grid.y > 65535) LLM_FAIL(-1, "lru_gates: too many column tiles");
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(lru_gates_kernel<T>, grid, 256, 0, stream, u, (const T*)ra, (const T*)ri, ra_bias, ri_bias, lam, decay_scale, a_out,
                   b_out, tokens, width, blocks);
        LLM_CHECK_LAUNCH("lru_gates");
        return 0;
    });
}

// longest: the most tokens a request brings (chooses the walk or the segments); scratch: float32 [2 * requests * segments * width]
// with segments = ceil(longest / llm_lru_segment()), needed when longest > llm_lru_segment().
LLM_API int llm_lru_scan(const float* a, const float* b, const void* proj, int ld, int y_col, int x_col, const float* bias_y,
                         const float* bias_x, int taps, float* state, const int* state_slots, const int* cu_seqlens, void* out,
                         int dtype, int requests, int width, int longest, int write, float* scratch, cudaStream_t stream) {
    if (requests == 0 || longest == 0) return 0;
    if (taps < 1) LLM_FAIL(-1, "lru_scan: %d taps", taps);
    const unsigned cb = (unsigned)((width + 127) / 128);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        if (longest <= kSegment) {
            llm_launch(lru_scan_walk_kernel<T>, dim3(cb, (unsigned)requests), 128, 0, stream, a, b, (const T*)proj, ld, y_col, x_col, bias_y,
                       bias_x, taps, state, state_slots, cu_seqlens, (T*)out, width, write);
            LLM_CHECK_LAUNCH("lru_scan");
            return 0;
        }
        if (!scratch) LLM_FAIL(-1, "lru_scan: segments need scratch");
        const int segments = (longest + kSegment - 1) / kSegment;
        if ((long long)requests * segments > 65535) LLM_FAIL(-1, "lru_scan: too many segments");
        float* seg_a = scratch;
        float* seg_b = scratch + (size_t)requests * segments * width;
        llm_launch(lru_segment_sums_kernel, dim3(cb, (unsigned)(requests * segments)), 128, 0, stream, a, b, cu_seqlens, seg_a, seg_b, width,
                   segments);
        LLM_CHECK_LAUNCH("lru_segment_sums");
        llm_launch(lru_segment_starts_kernel<T>, dim3(cb, (unsigned)requests), 128, 0, stream, (const float*)seg_a, seg_b, (const T*)proj, ld,
                   x_col, bias_x, taps, state, state_slots, cu_seqlens, width, segments, write);
        LLM_CHECK_LAUNCH("lru_segment_starts");
        llm_launch(lru_segment_apply_kernel<T>, dim3(cb, (unsigned)(requests * segments)), 128, 0, stream, a, b, (const float*)seg_b,
                   (const T*)proj, ld, y_col, bias_y, cu_seqlens, (T*)out, width, segments);
        LLM_CHECK_LAUNCH("lru_segment_apply");
        return 0;
    });
}

// A step of single tokens (every request brings one, or none): all of the above in one launch.  Sizes as in the three entry points.
LLM_API int llm_lru_step(const void* proj, int ld, int y_col, int x_col, const float* bias_y, const float* bias_x, const float* taps_w,
                         const float* conv_bias, int taps, const void* ra, const void* ri, const float* ra_bias, const float* ri_bias,
                         const float* lam, float decay_scale, float* state, const int* state_slots, const int* cu_seqlens, void* out,
                         int dtype, int requests, int width, int blocks, int write, cudaStream_t stream) {
    if (requests == 0) return 0;
    if (taps < 1) LLM_FAIL(-1, "lru_step: %d taps", taps);
    if (blocks < 1 || width % blocks) LLM_FAIL(-1, "lru_step: width %d is not a multiple of %d blocks", width, blocks);
    if (requests > 65535) LLM_FAIL(-1, "lru_step: too many requests");
    const size_t smem = (size_t)(width / blocks) * sizeof(float);
    if (smem > 200 * 1024) LLM_FAIL(-1, "lru_step: a gate block of %d channels does not fit shared memory", width / blocks);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        if (smem > 48 * 1024) cudaFuncSetAttribute(lru_step_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        llm_launch(lru_step_kernel<T>, dim3((unsigned)blocks, (unsigned)requests), width / blocks >= 128 ? 1024 : 256, smem, stream, (const T*)proj, ld, y_col, x_col, bias_y,
                   bias_x, taps_w, conv_bias, taps, (const T*)ra, (const T*)ri, ra_bias, ri_bias, lam, decay_scale, state, state_slots,
                   cu_seqlens, (T*)out, width, blocks, write);
        LLM_CHECK_LAUNCH("lru_step");
        return 0;
    });
}

LLM_TRACE_EXPORT(lru)
