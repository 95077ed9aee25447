// Grouped matrix products: many small products y_g = x_g . W_g^T in one launch, each group with a weight matrix of its own.
//
// Two ways to say which rows belong to which group:
//   uniform   every group multiplies the same `M` rows; group g reads its k-columns at a_offset + g * a_group_stride of the
//             row (per-head products on slices of one projection: a_group_stride = a head's width) or a whole other block
//             of rows (a_group_stride = rows * lda), and writes its n columns at c_offset + g * c_group_stride.
//   listed    a device list of tiles (group, first row, rows) over rows that were sorted by group beforehand (the experts
//             of a routed feed-forward: llm_moe_plan writes the list and its count, so nothing comes back to the host);
//             a row may be read through an index (`row_src`: sorted row -> token), the result row is the sorted row.
// Epilogue "glu": W_g holds n gate rows and then n up rows, and the [rows, 2n] intermediate never exists.  Form 1: the result is
// g * sigmoid(slope * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit).  Form 2: silu(w g) * (w u) with a
// weight w per sorted row (null: 1), which is the product of the row scaled by w since the product is linear in the row.
// Epilogue "out_gate" (without glu): every result number times the sigmoid of the float32 number at its place in a matrix laid out
// like the result.
//
// bfloat16: mma.sync m16n8k16 with float32 accumulators, tiles of 64 rows x 64 columns x 32 k, four warps; float32: FMA
// on the CUDA cores, no tensor cores, no TF32.  Every output element is summed over k in one fixed order, so a row's result
// does not depend on its group's other rows.  Sizes need not be multiples of anything (ragged edges are zero-filled; 16-byte
// loads are used when every row start allows them).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64;

struct GroupedArgs {
    const void* A; long long lda, a_group_stride, a_offset; const int* row_src;
    const void* W; long long w_group_stride;
    void* C; long long ldc, c_group_stride, c_offset;
    int M, N, K, groups, m_tiles;
    const int* tiles;          // listed mode: tiles[0] = count, entry i at tiles[4 + 4 * i] = (group, first row, rows, -)
    int glu; float limit, slope;
    const float* row_scale;    // form 2 of the glu epilogue: a factor per result row
    const float* out_gate;     // float32 laid out like C (same ldc and offsets): the result is multiplied by its sigmoid
    int vec_a, vec_w;
};

struct Tile { int group, row0, rows; bool live; };

__device__ __forceinline__ Tile resolve_tile(const GroupedArgs& a) {
    Tile t;
    if (a.tiles) {
        t.live = (int)blockIdx.y < a.tiles[0];
        const int* e = a.tiles + 4 + 4 * blockIdx.y;
        t.group = t.live ? e[0] : 0; t.row0 = t.live ? e[1] : 0; t.rows = t.live ? e[2] : 0;
    } else {
        t.group = blockIdx.y / a.m_tiles;
        t.row0 = (blockIdx.y % a.m_tiles) * BM;
        t.rows = min(BM, a.M - t.row0);
        t.live = t.rows > 0;
    }
    return t;
}

template <typename T>
__device__ __forceinline__ const T* a_row(const GroupedArgs& a, const Tile& t, int r) {
    const T* base = static_cast<const T*>(a.A);
    if (a.tiles) return base + (long long)(a.row_src ? a.row_src[t.row0 + r] : t.row0 + r) * a.lda;
    return base + a.a_offset + (long long)t.group * a.a_group_stride + (long long)(t.row0 + r) * a.lda;
}

__device__ __forceinline__ float glu(float g, float u, float limit, float slope) {
    if (limit < 0.f) {                  // form 2: `slope` carries the row's weight
        g *= slope;
        return g / (1.0f + expf(-g)) * (u * slope);
    }
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-slope * g)) * (u + 1.0f);
}

// ---- bfloat16 on the tensor cores -----------------------------------------------------------------------------
constexpr int BK16 = 32, PAD16 = 8;

// eight consecutive k of one row, zero beyond K or for a row that does not exist
__device__ __forceinline__ uint4 load8(const __nv_bfloat16* row, int k, int K, bool vec) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (!row || k >= K) return v;
    if (vec && k + 8 <= K) return *reinterpret_cast<const uint4*>(row + k);
    __nv_bfloat16 e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = k + i < K ? row[k + i] : __float2bfloat16(0.f);
    return *reinterpret_cast<uint4*>(e);
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <bool GLU>
__global__ void __launch_bounds__(128)
grouped_bf16_kernel(const GroupedArgs a) {
    pdl_trigger();
    pdl_wait();
    using bf16 = __nv_bfloat16;
    __shared__ __align__(16) bf16 As[BM][BK16 + PAD16];
    __shared__ __align__(16) bf16 Ws[GLU ? 2 : 1][BN][BK16 + PAD16];
    const Tile tile = resolve_tile(a);
    if (!tile.live) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    const int gq = lane >> 2, tq = lane & 3;
    const int n0 = blockIdx.x * BN;
    const bf16* Wg = static_cast<const bf16*>(a.W) + (long long)tile.group * a.w_group_stride;

    // loader: thread handles chunk c = tid, tid + 128 of 256 chunks (row = c / 4, k8 = (c % 4) * 8)
    const bf16* arow[2];
    const bf16* wrow[GLU ? 2 : 1][2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = (tid + i * 128) >> 2;
        arow[i] = r < tile.rows ? a_row<bf16>(a, tile, r) : nullptr;
#pragma unroll
        for (int s = 0; s < (GLU ? 2 : 1); ++s)
            wrow[s][i] = n0 + r < a.N ? Wg + ((long long)s * a.N + n0 + r) * a.K : nullptr;
    }
    float acc[GLU ? 2 : 1][2][4][4];
#pragma unroll
    for (int s = 0; s < (GLU ? 2 : 1); ++s)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[s][i][j][e] = 0.f;

    uint4 ra[2], rw[GLU ? 2 : 1][2];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int k = k0 + ((tid + i * 128) & 3) * 8;
            ra[i] = load8(arow[i], k, a.K, a.vec_a);
#pragma unroll
            for (int s = 0; s < (GLU ? 2 : 1); ++s) rw[s][i] = load8(wrow[s][i], k, a.K, a.vec_w);
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < a.K; k0 += BK16) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int c = tid + i * 128, r = c >> 2, kk = (c & 3) * 8;
            *reinterpret_cast<uint4*>(&As[r][kk]) = ra[i];
#pragma unroll
            for (int s = 0; s < (GLU ? 2 : 1); ++s) *reinterpret_cast<uint4*>(&Ws[s][r][kk]) = rw[s][i];
        }
        __syncthreads();
        if (k0 + BK16 < a.K) fetch(k0 + BK16);
#pragma unroll
        for (int ks = 0; ks < BK16; ks += 16) {
            uint32_t fa[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = wm + i * 16 + gq;
                fa[i][0] = *reinterpret_cast<const uint32_t*>(&As[r][ks + 2 * tq]);
                fa[i][1] = *reinterpret_cast<const uint32_t*>(&As[r + 8][ks + 2 * tq]);
                fa[i][2] = *reinterpret_cast<const uint32_t*>(&As[r][ks + 2 * tq + 8]);
                fa[i][3] = *reinterpret_cast<const uint32_t*>(&As[r + 8][ks + 2 * tq + 8]);
            }
#pragma unroll
            for (int s = 0; s < (GLU ? 2 : 1); ++s)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t fb[2];
                    const int n = wn + j * 8 + gq;
                    fb[0] = *reinterpret_cast<const uint32_t*>(&Ws[s][n][ks + 2 * tq]);
                    fb[1] = *reinterpret_cast<const uint32_t*>(&Ws[s][n][ks + 2 * tq + 8]);
#pragma unroll
                    for (int i = 0; i < 2; ++i) mma_bf16(acc[s][i][j], fa[i], fb);
                }
        }
        __syncthreads();
    }
    bf16* C = static_cast<bf16*>(a.C) + a.c_offset + (a.tiles ? 0 : (long long)tile.group * a.c_group_stride);
    const float* G = a.out_gate ? a.out_gate + a.c_offset + (a.tiles ? 0 : (long long)tile.group * a.c_group_stride) : nullptr;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = wm + i * 16 + gq + (e >> 1) * 8, n = n0 + wn + j * 8 + 2 * tq + (e & 1);
                if (r < tile.rows && n < a.N) {
                    float v = acc[0][i][j][e];
                    if (GLU) v = glu(v, acc[GLU ? 1 : 0][i][j][e], a.glu == 2 ? -1.f : a.limit,
                                     a.glu == 2 ? (a.row_scale ? a.row_scale[tile.row0 + r] : 1.f) : a.slope);
                    if (!GLU && G) v /= 1.0f + expf(-G[(long long)(tile.row0 + r) * a.ldc + n]);
                    C[(long long)(tile.row0 + r) * a.ldc + n] = __float2bfloat16_rn(v);
                }
            }
}

// The same product with its operands streamed by cp.async through a ring of stages (k-blocks of 64): what the experts' products of
// a decode step need, where a tile's few rows meet 64 weight rows of the whole k range and the kernel is bound by how many
// bytes it keeps in flight.  Taken when every 16-byte piece is aligned (else the kernel above runs).
constexpr int BKP = 64, PADP = 8, STAGES = 3;

template <bool GLU>
__global__ void __launch_bounds__(128)
grouped_bf16_pipe_kernel(const GroupedArgs a) {
    pdl_trigger();
    pdl_wait();
    using bf16 = __nv_bfloat16;
    constexpr int LD = BKP + PADP, NW = GLU ? 2 : 1;
    extern __shared__ __align__(16) unsigned char grouped_smem[];
    bf16* As = reinterpret_cast<bf16*>(grouped_smem);                      // [STAGES][BM][LD]
    bf16* Ws = As + (size_t)STAGES * BM * LD;                              // [STAGES][NW][BN][LD]
    const Tile tile = resolve_tile(a);
    if (!tile.live) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    const int gq = lane >> 2, tq = lane & 3;
    const int n0 = blockIdx.x * BN;
    const bf16* Wg = static_cast<const bf16*>(a.W) + (long long)tile.group * a.w_group_stride;
    // loader: thread (row = tid / 2, half = tid % 2) copies four 16-byte pieces of its row per operand and k-block
    const int lrow = tid >> 1, lhalf = (tid & 1) * 32;
    const bf16* arow = lrow < tile.rows ? a_row<bf16>(a, tile, lrow) : nullptr;
    const bf16* wrow[NW];
#pragma unroll
    for (int s = 0; s < NW; ++s) wrow[s] = n0 + lrow < a.N ? Wg + ((long long)s * a.N + n0 + lrow) * a.K : nullptr;
    const bf16* any = static_cast<const bf16*>(a.W);
    auto issue = [&](int kb, int stage) {
        const int k0 = kb * BKP + lhalf;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int k = k0 + c * 8;
            const int ab = arow && k < a.K ? 16 : 0;
            const uint32_t adst = (uint32_t)__cvta_generic_to_shared(As + ((size_t)stage * BM + lrow) * LD + lhalf + c * 8);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(adst), "l"(ab ? arow + k : any), "r"(ab) : "memory");
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                const int wb = wrow[s] && k < a.K ? 16 : 0;
                const uint32_t wdst = (uint32_t)__cvta_generic_to_shared(Ws + (((size_t)stage * NW + s) * BN + lrow) * LD + lhalf + c * 8);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(wdst), "l"(wb ? wrow[s] + k : any), "r"(wb) : "memory");
            }
        }
    };
    float acc[NW][2][4][4];
#pragma unroll
    for (int s = 0; s < NW; ++s)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[s][i][j][e] = 0.f;
    const int k_blocks = (a.K + BKP - 1) / BKP;
#pragma unroll
    for (int p = 0; p < STAGES - 1; ++p) {
        if (p < k_blocks) issue(p, p);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kb = 0; kb < k_blocks; ++kb) {
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
        __syncthreads();                                   // k-block kb has landed for all; the stage refilled below was used up
        if (kb + STAGES - 1 < k_blocks) issue(kb + STAGES - 1, (kb + STAGES - 1) % STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const bf16* Ab = As + (size_t)(kb % STAGES) * BM * LD;
        const bf16* Wb = Ws + (size_t)(kb % STAGES) * NW * BN * LD;
#pragma unroll
        for (int ks = 0; ks < BKP; ks += 16) {
            uint32_t fa[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const bf16* r0 = Ab + (size_t)(wm + i * 16 + gq) * LD + ks + 2 * tq;
                fa[i][0] = *reinterpret_cast<const uint32_t*>(r0);
                fa[i][1] = *reinterpret_cast<const uint32_t*>(r0 + 8 * LD);
                fa[i][2] = *reinterpret_cast<const uint32_t*>(r0 + 8);
                fa[i][3] = *reinterpret_cast<const uint32_t*>(r0 + 8 * LD + 8);
            }
#pragma unroll
            for (int s = 0; s < NW; ++s)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t fb[2];
                    const bf16* c0 = Wb + ((size_t)s * BN + wn + j * 8 + gq) * LD + ks + 2 * tq;
                    fb[0] = *reinterpret_cast<const uint32_t*>(c0);
                    fb[1] = *reinterpret_cast<const uint32_t*>(c0 + 8);
#pragma unroll
                    for (int i = 0; i < 2; ++i) mma_bf16(acc[s][i][j], fa[i], fb);
                }
        }
    }
    bf16* C = static_cast<bf16*>(a.C) + a.c_offset + (a.tiles ? 0 : (long long)tile.group * a.c_group_stride);
    const float* G = a.out_gate ? a.out_gate + a.c_offset + (a.tiles ? 0 : (long long)tile.group * a.c_group_stride) : nullptr;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = wm + i * 16 + gq + (e >> 1) * 8, n = n0 + wn + j * 8 + 2 * tq + (e & 1);
                if (r < tile.rows && n < a.N) {
                    float v = acc[0][i][j][e];
                    if (GLU) v = glu(v, acc[NW - 1][i][j][e], a.glu == 2 ? -1.f : a.limit,
                                     a.glu == 2 ? (a.row_scale ? a.row_scale[tile.row0 + r] : 1.f) : a.slope);
                    if (!GLU && G) v /= 1.0f + expf(-G[(long long)(tile.row0 + r) * a.ldc + n]);
                    C[(long long)(tile.row0 + r) * a.ldc + n] = __float2bfloat16_rn(v);
                }
            }
}

// ---- float32 on the CUDA cores -------------------------------------------------------------------------------
constexpr int BK32 = 16, TM = 4, TN = 4;

template <bool GLU>
__global__ void __launch_bounds__(256)
grouped_f32_kernel(const GroupedArgs a) {
    pdl_trigger();
    pdl_wait();
    __shared__ float As[BK32][BM + 4];
    __shared__ float Ws[GLU ? 2 : 1][BK32][BN + 4];
    const Tile tile = resolve_tile(a);
    if (!tile.live) return;
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * BN;
    const int tr = tid / 16, tc = tid % 16;
    const int lrow = tid / 4, lk = (tid % 4) * 4;
    const float* Wg = static_cast<const float*>(a.W) + (long long)tile.group * a.w_group_stride;
    const float* arow = lrow < tile.rows ? a_row<float>(a, tile, lrow) : nullptr;
    const float* wrow[GLU ? 2 : 1];
#pragma unroll
    for (int s = 0; s < (GLU ? 2 : 1); ++s) wrow[s] = n0 + lrow < a.N ? Wg + ((long long)s * a.N + n0 + lrow) * a.K : nullptr;
    auto load4 = [&](const float* row, int k, bool vec) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (!row || k >= a.K) return v;
        if (vec && k + 4 <= a.K) return *reinterpret_cast<const float4*>(row + k);
        v.x = row[k];
        if (k + 1 < a.K) v.y = row[k + 1];
        if (k + 2 < a.K) v.z = row[k + 2];
        if (k + 3 < a.K) v.w = row[k + 3];
        return v;
    };
    float acc[GLU ? 2 : 1][TM][TN];
#pragma unroll
    for (int s = 0; s < (GLU ? 2 : 1); ++s)
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[s][i][j] = 0.f;
    for (int k0 = 0; k0 < a.K; k0 += BK32) {
        {
            const float4 v = load4(arow, k0 + lk, a.vec_a);
            As[lk][lrow] = v.x; As[lk + 1][lrow] = v.y; As[lk + 2][lrow] = v.z; As[lk + 3][lrow] = v.w;
        }
#pragma unroll
        for (int s = 0; s < (GLU ? 2 : 1); ++s) {
            const float4 v = load4(wrow[s], k0 + lk, a.vec_w);
            Ws[s][lk][lrow] = v.x; Ws[s][lk + 1][lrow] = v.y; Ws[s][lk + 2][lrow] = v.z; Ws[s][lk + 3][lrow] = v.w;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK32; ++k) {
            float av[TM], bv[GLU ? 2 : 1][TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = As[k][tr * TM + i];
#pragma unroll
            for (int s = 0; s < (GLU ? 2 : 1); ++s)
#pragma unroll
                for (int j = 0; j < TN; ++j) bv[s][j] = Ws[s][k][tc * TN + j];
#pragma unroll
            for (int s = 0; s < (GLU ? 2 : 1); ++s)
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) acc[s][i][j] = fmaf(av[i], bv[s][j], acc[s][i][j]);
        }
        __syncthreads();
    }
    float* C = static_cast<float*>(a.C) + a.c_offset + (a.tiles ? 0 : (long long)tile.group * a.c_group_stride);
    const float* G = a.out_gate ? a.out_gate + a.c_offset + (a.tiles ? 0 : (long long)tile.group * a.c_group_stride) : nullptr;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = tr * TM + i;
        if (r >= tile.rows) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tc * TN + j;
            if (n >= a.N) continue;
            float v = acc[0][i][j];
            if (GLU) v = glu(v, acc[GLU ? 1 : 0][i][j], a.glu == 2 ? -1.f : a.limit,
                             a.glu == 2 ? (a.row_scale ? a.row_scale[tile.row0 + r] : 1.f) : a.slope);
            if (!GLU && G) v /= 1.0f + expf(-G[(long long)(tile.row0 + r) * a.ldc + n]);
            C[(long long)(tile.row0 + r) * a.ldc + n] = v;
        }
    }
}

}  // namespace

// Rows a tile of the listed form holds (llm_moe_plan cuts the sorted rows into tiles of this many).
LLM_API int llm_gemm_grouped_tile_rows() { return BM; }

// A, W, C of `dtype`.  Uniform form: tiles == null, `groups` groups of `M` rows.  Listed form: tiles != null (device:
// tiles[0] = count, then four ints per tile), `max_tiles` bounds the count, a_offset / a_group_stride / c_group_stride unused.
// W: [groups, N (2N with glu), K] contiguous.
LLM_API int llm_gemm_grouped(const void* A, long long lda, long long a_group_stride, long long a_offset, const int* row_src,
                             const void* W, void* C, long long ldc, long long c_group_stride, long long c_offset, int dtype,
                             int M, int N, int K, int groups, const int* tiles, int max_tiles, int glu, float limit, float slope,
                             const float* row_scale, const float* out_gate, cudaStream_t stream) {
    if (N <= 0 || K <= 0 || groups <= 0) return 0;
    if (!tiles && M <= 0) return 0;
    if (tiles && max_tiles <= 0) return 0;
    GroupedArgs a;
    a.A = A; a.lda = lda; a.a_group_stride = a_group_stride; a.a_offset = a_offset; a.row_src = row_src;
    a.W = W; a.w_group_stride = (long long)(glu ? 2 : 1) * N * K;
    a.C = C; a.ldc = ldc; a.c_group_stride = c_group_stride; a.c_offset = c_offset;
    a.M = M; a.N = N; a.K = K; a.groups = groups; a.m_tiles = tiles ? 0 : (M + BM - 1) / BM;
    a.tiles = tiles; a.glu = glu; a.limit = limit; a.slope = slope; a.row_scale = row_scale; a.out_gate = out_gate;
    if (out_gate && glu) LLM_FAIL(-1, "gemm_grouped: an output gate and a glu epilogue exclude one another");
    if (glu < 0 || glu > 2) LLM_FAIL(-1, "gemm_grouped: glu form %d is not known", glu);
    if (glu == 1 && limit < 0.f) LLM_FAIL(-1, "gemm_grouped: the clamp's limit %g is negative", (double)limit);
    const int per = dtype == LLM_BF16 ? 8 : 4;
    a.vec_a = !(lda % per) && !(a_group_stride % per) && !(a_offset % per) && !((uintptr_t)A & 15);
    a.vec_w = !(K % per) && !((uintptr_t)W & 15);
    const long long rows_y = tiles ? max_tiles : (long long)a.m_tiles * groups;
    if (rows_y > 65535) LLM_FAIL(-1, "gemm_grouped: %lld row tiles are too many for one launch", rows_y);
    dim3 grid((N + BN - 1) / BN, (unsigned)rows_y);
    // few rows a group (decode steps): the streamed form; many rows: the plain tiles re-use their operands enough and run faster
    const long long rows_about = tiles ? (long long)(max_tiles - groups) * BM : M;
    if (dtype == LLM_BF16 && a.vec_a && a.vec_w && rows_about <= 1024) {
        const size_t smem = (size_t)STAGES * (BM + (glu ? 2 : 1) * BN) * (BKP + PADP) * 2;
        if (glu) {
            cudaFuncSetAttribute(grouped_bf16_pipe_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            llm_launch(grouped_bf16_pipe_kernel<true>, grid, 128, smem, stream, a);
        } else {
            cudaFuncSetAttribute(grouped_bf16_pipe_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            llm_launch(grouped_bf16_pipe_kernel<false>, grid, 128, smem, stream, a);
        }
    } else if (dtype == LLM_BF16) {
        if (glu) llm_launch(grouped_bf16_kernel<true>, grid, 128, 0, stream, a);
        else llm_launch(grouped_bf16_kernel<false>, grid, 128, 0, stream, a);
    } else if (dtype == LLM_F32) {
        if (glu) llm_launch(grouped_f32_kernel<true>, grid, 256, 0, stream, a);
        else llm_launch(grouped_f32_kernel<false>, grid, 256, 0, stream, a);
    } else {
        LLM_FAIL(-1, "gemm_grouped: unknown dtype code %d", dtype);
    }
    LLM_CHECK_LAUNCH("gemm_grouped");
    return 0;
}

LLM_TRACE_EXPORT(gemm_grouped)
