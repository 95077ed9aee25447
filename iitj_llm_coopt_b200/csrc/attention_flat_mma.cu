// Attention over flat-page caches on the tensor cores (bfloat16; see attention_flat.cu for the cache layout and the
// one-warp-per-row form that serves float32 and sizes this kernel does not take).
//
// A block takes 64 rows, a row being one (query token, query head) pair: up to 64 / heads_per_block neighbouring tokens of one
// request times the heads of one key/value head's group (a group of more than 64 heads is cut into blocks of 64).  All rows
// of a block share their keys and values, so a tile of 32 keys travels to shared memory once and serves every row: with one
// latent row per token and 32 heads that is 32 times less traffic than a warp per row.  Tiles arrive by cp.async into two
// stages, one tile ahead of the arithmetic.  Per key tile (of 32 keys, or of 16 where two blocks with tiles of 32 would not fit an
// SM's shared memory; tiles start at multiples of their size of the key position): S = Q K^T by mma.sync m16n8k16 (a warp owns 16 rows), mask and running softmax in float32
// registers, P rounded to bfloat16 only as the operand of P V, V fragments by ldmatrix.trans from the row-major tile, O in
// float32 registers.  A value head wider than 256 is cut into slices of 256 over blockIdx.z (each slice's blocks recompute
// S).  With `splits` > 1 a block walks only its share of the key tiles and leaves (O, m, l) for the merge kernel, so a few
// decoded tokens over long contexts still fill the GPU.  Rows of a tile that no query of the tile can see are never read
// from the cache (they may lie in pages a window has given back).
#include "common.cuh"

namespace {

constexpr int kRows = 64, kPad = 8;

// Keys of a tile: 32, or 16 where 32 would leave room for one block an SM only (rows of several hundred numbers).
static inline size_t flat_smem_bytes(int key_dim, int slice_w, int shared_value, int keys) {
    return ((size_t)(kRows + 2 * keys) * (key_dim + kPad) + (shared_value ? 0 : (size_t)2 * keys * (slice_w + kPad))) * 2;
}

// Width of a block's slice of the value head: wider slices recompute the scores less often but hold more of O in registers.
static inline int slice_width(int value_dim) { return value_dim <= 64 ? 64 : value_dim <= 128 ? 128 : 256; }

struct FlatMmaArgs {
    const __nv_bfloat16* q; int q_stride;
    const __nv_bfloat16* cache; long long page_stride;
    const int* block_table; int table_width;
    const int* tiles; int n_tiles;            // (first token row, tokens, position of the first, request)
    const float* gate; int gate_cols;         // one gate number per head (1) or per output number (value_dim)
    const float* slopes;                      // per head: slope * (query position - key position) is taken off the score
    const float* sinks;                       // per head: exp(sink) joins every row's denominator once, without a value (null: none)
    float softcap, temp_coef; int temp_every; // score squashing and query temperature (0: none), as in attention_flat.cu
    __nv_bfloat16* out; int out_stride;
    float* part_o; float* part_ml;            // [token, head, split, value_dim] and [token, head, split, 2] when splits > 1
    int heads, kv_heads, key_dim, value_dim, shared_value, page_size, window, heads_per_block, tokens_per_tile, splits;
    float scale;
};

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int NT, int kKeys>      // NT: n-tiles of 8 value dims a block's slice holds (32: slices of 256, 16: of 128, 8: of 64)
__global__ void __launch_bounds__(128)
attention_flat_mma_kernel(const FlatMmaArgs a) {
    pdl_trigger();
    pdl_wait();
    using bf16 = __nv_bfloat16;
    extern __shared__ __align__(16) unsigned char flat_smem[];
    const int kd = a.key_dim, ldk = kd + kPad;
    const int slice_w = NT * 8, ldv = slice_w + kPad;
    bf16* Qs = reinterpret_cast<bf16*>(flat_smem);                     // [64][ldk]
    bf16* Ks0 = Qs + (size_t)kRows * ldk;                              // two stages of [32][ldk]
    bf16* Vs0 = Ks0 + (size_t)2 * kKeys * ldk;                         // two stages of [32][ldv], unused with shared values

    const int tile = blockIdx.x / a.splits, split = blockIdx.x % a.splits;
    const int* rec = a.tiles + 4 * tile;
    const int row0 = rec[0], ntok = rec[1], pos0 = rec[2], req = rec[3];
    const int group = a.heads / a.kv_heads, hpb = a.heads_per_block, head_blocks = (group + hpb - 1) / hpb;
    const int kvh = blockIdx.y / head_blocks, hb = blockIdx.y % head_blocks;
    const int slice0 = blockIdx.z * slice_w;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
    const int* table = a.block_table + (size_t)req * a.table_width;

    // the tile's key range and this split's share of its key tiles
    const int kmax = pos0 + ntok - 1;
    const int kmin = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int first_tile = kmin / kKeys, n_ktiles = kmax / kKeys - first_tile + 1;
    const int per_split = (n_ktiles + a.splits - 1) / a.splits;
    const int kt_lo = first_tile + split * per_split, kt_hi = min(first_tile + n_ktiles, kt_lo + per_split);

    // queries: row r = token r / hpb, head hb * hpb + r % hpb of the group
    const int chunks = kd / 8;
    for (int c = tid; c < kRows * chunks; c += 128) {
        const int r = c / chunks, k8 = (c % chunks) * 8;
        const int ti = r / hpb, hg = hb * hpb + r % hpb;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (ti < ntok && hg < group)
            v = *reinterpret_cast<const uint4*>(a.q + (size_t)(row0 + ti) * a.q_stride + (size_t)(kvh * group + hg) * kd + k8);
        *reinterpret_cast<uint4*>(Qs + (size_t)r * ldk + k8) = v;
    }
    // this thread's two rows (gq and gq + 8 of the warp's 16)
    int row_pos[2], row_lo[2];
    float row_scale[2], row_slope[2];
    bool row_ok[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int r = warp * 16 + gq + e * 8;
        const int ti = r / hpb, hg = hb * hpb + r % hpb;
        row_ok[e] = ti < ntok && hg < group;
        row_pos[e] = pos0 + ti;
        row_lo[e] = a.window > 0 ? max(0, row_pos[e] - a.window + 1) : 0;
        row_scale[e] = a.temp_every > 0 ? a.scale * (1.0f + a.temp_coef * logf((float)((row_pos[e] + 1) / a.temp_every) + 1.0f)) : a.scale;
        row_slope[e] = a.slopes && row_ok[e] ? a.slopes[kvh * group + hg] : 0.f;
    }
    const float inv_cap = a.softcap > 0.f ? 1.0f / a.softcap : 0.f;
    const bool warp_live = (warp * 16) / hpb < ntok;
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    const size_t key_head = (size_t)kvh * a.page_size * kd;
    const size_t value_plane = (size_t)a.kv_heads * a.page_size * kd + (size_t)kvh * a.page_size * a.value_dim;
    const int vchunks = slice_w / 8;

    // Key (and value) tiles arrive by cp.async, one tile ahead of the arithmetic: thread (row = tid / 4, quarter = tid % 4)
    // copies every fourth 16-byte piece of its row, so it looks up one page per tile; a row that no query of the tile sees
    // is filled with zeros (copy of zero bytes).
    constexpr int LT = 128 / kKeys;                        // threads that share a row's copies
    const int lrow = tid / LT, lq = tid % LT;
    auto issue = [&](int kt, int stage) {
        const int j = kt * kKeys + lrow;
        const bool live = j >= kmin && j <= kmax;
        const bf16* page = a.cache + (live ? (size_t)table[j / a.page_size] * a.page_stride : 0);
        const bf16* ksrc = page + (live ? key_head + (size_t)(j % a.page_size) * kd : 0);
        bf16* kdst = Ks0 + (size_t)stage * kKeys * ldk + (size_t)lrow * ldk;
        const int bytes = live ? 16 : 0;
        for (int c = lq; c < chunks; c += LT) {
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(kdst + c * 8);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(ksrc + c * 8), "r"(bytes) : "memory");
        }
        if (!a.shared_value) {
            const bf16* vsrc = page + (live ? value_plane + (size_t)(j % a.page_size) * a.value_dim + slice0 : 0);
            bf16* vdst = Vs0 + (size_t)stage * kKeys * ldv + (size_t)lrow * ldv;
            for (int c = lq; c < vchunks; c += LT) {
                const int vb = live && slice0 + c * 8 < a.value_dim ? 16 : 0;
                const uint32_t dst = (uint32_t)__cvta_generic_to_shared(vdst + c * 8);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(vb ? vsrc + c * 8 : a.cache), "r"(vb) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (kt_lo < kt_hi) issue(kt_lo, 0);
    for (int kt = kt_lo; kt < kt_hi; ++kt) {
        const int k0 = kt * kKeys, stage = (kt - kt_lo) & 1;
        const bf16* Ks = Ks0 + (size_t)stage * kKeys * ldk;
        const bf16* Vs = Vs0 + (size_t)stage * kKeys * ldv;
        if (kt + 1 < kt_hi) {
            issue(kt + 1, stage ^ 1);                      // (the stage it overwrites was used up before the barrier below, last round)
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                                   // this tile has landed for every thread (and Qs is written, first time)
        // S = Q K^T for the warp's 16 rows and the tile's 32 keys (a warp whose rows all lie beyond the tile's tokens, as half
        // of them do for one decoded token of 32 heads, only helps with the copies and the barriers)
        if (warp_live) {
        constexpr int KB = kKeys / 8;                      // blocks of 8 keys
        float s[KB][4];
#pragma unroll
        for (int j = 0; j < KB; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
        // fragments by ldmatrix.x4: the left operand's four 8x8 pieces of 16 rows x 16 dims at once, and the right operand's
        // pieces of two blocks of 8 keys at once (a key tile's rows are the product's columns as they lie)
        const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(
            Qs + (size_t)(warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * ldk + (lane >> 4) * 8);
        const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(
            Ks + (size_t)((lane >> 4) * 8 + (lane & 7)) * ldk + ((lane >> 3) & 1) * 8);
        for (int ks = 0; ks < kd; ks += 16) {
            uint32_t fa[4], fb[4];
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(fa[0]), "=r"(fa[1]), "=r"(fa[2]), "=r"(fa[3]) : "r"(q_addr + ks * 2));
#pragma unroll
            for (int jj = 0; jj < KB / 2; ++jj) {
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(fb[0]), "=r"(fb[1]), "=r"(fb[2]), "=r"(fb[3]) : "r"(k_addr + (jj * 16 * ldk + ks) * 2));
                mma16816(s[2 * jj], fa, fb[0], fb[1]);
                mma16816(s[2 * jj + 1], fa, fb[2], fb[3]);
            }
        }
        // mask, running softmax (each row's 32 scores sit in the four lanes of a quad)
        float corr[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < KB; ++j)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int key = k0 + j * 8 + 2 * tq + c;
                    const bool seen = row_ok[e] && key <= row_pos[e] && key >= row_lo[e];
                    float v = s[j][2 * e + c] * row_scale[e];
                    if (a.softcap > 0.f) v = a.softcap * tanhf(v * inv_cap);
                    v = seen ? v - row_slope[e] * (float)(row_pos[e] - key) : -INFINITY;
                    s[j][2 * e + c] = v;
                    mx = fmaxf(mx, v);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[e], mx);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            corr[e] = expf(m[e] - m_use);                     // 0 while the row has seen nothing
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < KB; ++j)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const float p = expf(s[j][2 * e + c] - m_use);
                    s[j][2 * e + c] = p;
                    sum += p;
                }
            l[e] = l[e] * corr[e] + sum;
            m[e] = m_new;
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
        }
        // O += P V: P's accumulator layout of two neighbouring key blocks of 8 is the left operand's layout of 16 keys
        const bf16* vbase = a.shared_value ? Ks + slice0 : Vs;
        const int ldvv = a.shared_value ? ldk : ldv;
#pragma unroll
        for (int kk = 0; kk < KB / 2; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            const bf16* vrow = vbase + (size_t)(kk * 16 + (lane & 15)) * ldvv;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                if (slice0 + n * 8 < a.value_dim) {          // the same for the whole warp
                    uint32_t b0, b1;
                    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(vrow + n * 8);
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                    mma16816(o[n], pa, b0, b1);
                }
            }
        }
        }
        __syncthreads();                                   // every warp is done with this stage before it is refilled
    }
    // results
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        l[e] += __shfl_xor_sync(0xffffffffu, l[e], 1);
        l[e] += __shfl_xor_sync(0xffffffffu, l[e], 2);
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        if (!row_ok[e]) continue;
        const int r = warp * 16 + gq + e * 8;
        const int t = row0 + r / hpb, head = kvh * group + hb * hpb + r % hpb;
        if (a.splits == 1) {
            if (a.sinks) l[e] += expf(a.sinks[head] - m[e]);
            float inv = 1.0f / l[e];
            if (a.gate && a.gate_cols == 1) inv *= 1.0f / (1.0f + expf(-a.gate[(size_t)t * a.heads + head]));
            const float* grow = a.gate && a.gate_cols > 1 ? a.gate + ((size_t)t * a.heads + head) * a.value_dim + slice0 : nullptr;
            bf16* dst = a.out + (size_t)t * a.out_stride + (size_t)head * a.value_dim + slice0;
#pragma unroll
            for (int n = 0; n < NT; ++n)
                if (slice0 + n * 8 < a.value_dim) {
                    float g0 = inv, g1 = inv;
                    if (grow) {
                        const float2 g = *reinterpret_cast<const float2*>(grow + n * 8 + 2 * tq);
                        g0 = inv / (1.0f + expf(-g.x));
                        g1 = inv / (1.0f + expf(-g.y));
                    }
                    *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * tq) = pack_bf16(o[n][2 * e] * g0, o[n][2 * e + 1] * g1);
                }
        } else {
            const size_t item = ((size_t)t * a.heads + head) * a.splits + split;
            float* dst = a.part_o + item * a.value_dim + slice0;
#pragma unroll
            for (int n = 0; n < NT; ++n)
                if (slice0 + n * 8 < a.value_dim)
                    *reinterpret_cast<float2*>(dst + n * 8 + 2 * tq) = make_float2(o[n][2 * e], o[n][2 * e + 1]);
            if (tq == 0 && blockIdx.z == 0) {
                a.part_ml[item * 2] = m[e];
                a.part_ml[item * 2 + 1] = l[e];
            }
        }
    }
}

// out[t, head] = sum_s O_s e^(m_s - m) / sum_s l_s e^(m_s - m), times the gate; one block per (token, head).
__global__ void __launch_bounds__(128)
flat_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const float* __restrict__ gate, int gate_cols,
                  const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out, int out_stride, int heads, int value_dim, int splits) {
    pdl_trigger();
    pdl_wait();
    const size_t item = blockIdx.x;                       // token * heads + head
    const float* ml = part_ml + item * splits * 2;
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, ml[2 * s]);
    float l = 0.f;
    for (int s = 0; s < splits; ++s) l += ml[2 * s + 1] * (ml[2 * s] == -INFINITY ? 0.f : expf(ml[2 * s] - m));
    const size_t t = item / heads, h = item % heads;
    if (sinks) l += expf(sinks[h] - m);                   // once for the row, whatever the count of splits
    float inv = 1.0f / l;
    if (gate && gate_cols == 1) inv *= 1.0f / (1.0f + expf(-gate[item]));
    const float* grow = gate && gate_cols > 1 ? gate + item * value_dim : nullptr;
    for (int d = threadIdx.x; d < value_dim; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s)
            if (ml[2 * s] != -INFINITY) acc += part_o[(item * splits + s) * value_dim + d] * expf(ml[2 * s] - m);
        out[t * out_stride + h * value_dim + d] = __float2bfloat16_rn(grow ? acc * inv / (1.0f + expf(-grow[d])) : acc * inv);
    }
}

}  // namespace

// Sizes the tensor-core form takes: 16-byte rows everywhere and whole MMA tiles.
LLM_API int llm_attention_flat_mma_supported(int heads, int kv_heads, int key_dim, int value_dim, int shared_value,
                                             long long page_stride) {
    if (kv_heads <= 0 || heads % kv_heads) return 0;
    if (key_dim % 16 || value_dim % 8 || key_dim > 1024 || value_dim > 1024 || page_stride % 8) return 0;
    if (shared_value && value_dim > key_dim) return 0;
    const int slice_w = slice_width(value_dim);
    return flat_smem_bytes(key_dim, slice_w, shared_value, 16) <= 200 * 1024;
}

// Shared memory of one block in bytes (what bounds the blocks an SM holds at wide rows).
LLM_API int llm_attention_flat_mma_smem(int key_dim, int value_dim, int shared_value) {
    const int slice_w = slice_width(value_dim);
    const size_t wide = flat_smem_bytes(key_dim, slice_w, shared_value, 32);
    return (int)(2 * wide + 2048 <= 227 * 1024 ? wide : flat_smem_bytes(key_dim, slice_w, shared_value, 16));
}

// Heads of a group that one block takes (the rest of its 64 rows are neighbouring tokens).
LLM_API int llm_attention_flat_mma_heads_per_block(int heads, int kv_heads) {
    const int group = heads / (kv_heads > 0 ? kv_heads : 1);
    return group < kRows ? group : kRows;
}

// tiles [n_tiles, 4]: (first token row, tokens <= 64 / heads_per_block, position of the first, request).  splits > 1 needs
// part_o [tokens, heads, splits, value_dim] and part_ml [tokens, heads, splits, 2] float32 and runs the merge after.
LLM_API int llm_attention_flat_mma(const void* q, int q_stride, const void* cache, long long page_stride, const int* block_table,
                                   int table_width, const int* tiles, int n_tiles, const float* gate, int gate_cols, void* out,
                                   int out_stride, int tokens, int heads, int kv_heads, int key_dim, int value_dim, int shared_value,
                                   int page_size, int window, float scale, float softcap, const float* slopes, float temp_coef,
                                   int temp_every, int splits, float* part_o, float* part_ml, const float* sinks, cudaStream_t stream) {
    if (n_tiles == 0) return 0;
    if (!llm_attention_flat_mma_supported(heads, kv_heads, key_dim, value_dim, shared_value, page_stride))
        LLM_FAIL(-1, "attention_flat_mma: sizes not taken (key_dim %d, value_dim %d)", key_dim, value_dim);
    if (gate && gate_cols != 1 && gate_cols != value_dim)
        LLM_FAIL(-1, "attention_flat_mma: a gate has one number per head or one per output number (%d, value_dim %d)", gate_cols, value_dim);
    if (splits < 1) splits = 1;
    if (splits > 1 && (!part_o || !part_ml)) LLM_FAIL(-1, "attention_flat_mma: key splits need partial buffers");
    if (((uintptr_t)q & 15) || ((uintptr_t)cache & 15) || q_stride % 8) LLM_FAIL(-1, "attention_flat_mma: rows must start on 16 bytes");
    FlatMmaArgs a;
    a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride; a.cache = (const __nv_bfloat16*)cache; a.page_stride = page_stride;
    a.block_table = block_table; a.table_width = table_width; a.tiles = tiles; a.n_tiles = n_tiles; a.gate = gate;
    a.gate_cols = gate_cols; a.slopes = slopes; a.sinks = sinks; a.softcap = softcap; a.temp_coef = temp_coef; a.temp_every = temp_every;
    a.out = (__nv_bfloat16*)out; a.out_stride = out_stride; a.part_o = part_o; a.part_ml = part_ml;
    a.heads = heads; a.kv_heads = kv_heads; a.key_dim = key_dim; a.value_dim = value_dim; a.shared_value = shared_value;
    a.page_size = page_size; a.window = window; a.splits = splits; a.scale = scale;
    a.heads_per_block = llm_attention_flat_mma_heads_per_block(heads, kv_heads);
    a.tokens_per_tile = kRows / a.heads_per_block;
    const int group = heads / kv_heads, head_blocks = (group + a.heads_per_block - 1) / a.heads_per_block;
    const int slice_w = slice_width(value_dim);
    const int slices = (value_dim + slice_w - 1) / slice_w;
    // tiles of 32 keys unless two blocks of them do not fit an SM's shared memory: then tiles of 16
    const int keys = 2 * flat_smem_bytes(key_dim, slice_w, shared_value, 32) + 2048 <= 227 * 1024 ? 32 : 16;
    const size_t smem = flat_smem_bytes(key_dim, slice_w, shared_value, keys);
    dim3 grid((unsigned)n_tiles * splits, (unsigned)kv_heads * head_blocks, (unsigned)slices);
    if (grid.y > 65535) LLM_FAIL(-1, "attention_flat_mma: too many heads");
#define LLM_FLAT_MMA(NT, KEYS)                                                                                         \
    do {                                                                                                               \
        cudaFuncSetAttribute(attention_flat_mma_kernel<NT, KEYS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        llm_launch(attention_flat_mma_kernel<NT, KEYS>, grid, 128, smem, stream, a);                                   \
    } while (0)
    if (slice_w == 64) { if (keys == 32) LLM_FLAT_MMA(8, 32); else LLM_FLAT_MMA(8, 16); }
    else if (slice_w == 128) { if (keys == 32) LLM_FLAT_MMA(16, 32); else LLM_FLAT_MMA(16, 16); }
    else { if (keys == 32) LLM_FLAT_MMA(32, 32); else LLM_FLAT_MMA(32, 16); }
#undef LLM_FLAT_MMA
    LLM_CHECK_LAUNCH("attention_flat_mma");
    if (splits > 1) {
        llm_launch(flat_merge_kernel, (unsigned)(tokens * heads), 128, 0, stream, (const float*)part_o, (const float*)part_ml, gate,
                   gate_cols, sinks, (__nv_bfloat16*)out, out_stride, heads, value_dim, splits);
        LLM_CHECK_LAUNCH("attention_flat_merge");
    }
    return 0;
}

LLM_TRACE_EXPORT(attention_flat_mma)
