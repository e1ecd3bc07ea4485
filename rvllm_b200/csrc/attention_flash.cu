// Paged flash attention for bfloat16, prefill and decode from one template.
//
// The rows of a tile are (token, query head) pairs of ONE key/value head: the G = nh / nkv
// query heads that share a key/value head are packed into the row dimension, so every key and
// value is fetched once per group.  A CTA owns a tile of 16 * WARPS_M rows of one sequence and
// one kv head, and walks the keys in tiles of 64 through the sequence's block table:
//   prefill / mixed steps: WARPS_M = 4, WARPS_N = 1 - the four warps own 16 rows each;
//   decode (one token per sequence): WARPS_M = 1, WARPS_N = 4 - the warps share 16 rows and own
//     16 of the tile's 64 keys each; their partial results are merged through shared memory.
// The keys of a sequence can also be split over `num_splits` CTAs; each writes a partial
// (unnormalised sum, running maximum, denominator) to scratch memory and a second kernel merges
// them with the same algebra.  Scores, softmax and the weighted sum are in float; the two
// products run on the tensor cores (mma.sync m16n8k16, bf16 in, float accumulate).
//
// Rule (v3/kernels/paged_attention_sm89.cu:277-308 of the reference): a sequence's q_len tokens
// of this step are the tail of its ctx_len cached tokens; token i sits at position
// p = ctx_len - q_len + i and sees keys (p - window, p] (all of [0, p] without a window).
// Cache layer layout: [num_pages, 2 (k, v), nkv, page_size, HEAD_DIM], page_size a power of two.
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head_dim must be a multiple of 16 up to 256");

#define KV_TILE 64
#ifndef DECODE_STAGES
#define DECODE_STAGES 2     // cp.async stages of the decode tiling (more stages measured slower: fewer CTAs fit an SM)
#endif
#define TABLE_CACHE 1024   // block-table entries of a CTA's key range kept in shared memory
// a row of the shared-memory tiles is padded by 16 bytes: the stride is an odd multiple of
// 16 bytes, so the 8 rows an ldmatrix reads fall into different banks
#define ROW_BYTES (HEAD_DIM * 2 + 16)
#define TILE_BYTES (KV_TILE * ROW_BYTES)

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;     // src-size 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct FlashParams {
    const __nv_bfloat16* q;        // [n_tokens, nh, HEAD_DIM]
    const __nv_bfloat16* cache;    // one layer
    const int* block_tables;       // [num_seqs, max_blocks]
    const int* cu_seqlens;         // [num_seqs + 1]
    const int* ctx_lens;           // [num_seqs]
    __nv_bfloat16* out;            // [n_tokens, nh, HEAD_DIM]
    float* part_o;                 // [num_splits, n_tokens, nh, HEAD_DIM]   (num_splits > 1)
    float* part_ml;                // [num_splits, n_tokens, nh, 2]
    int n_tokens, nh, nkv, page_shift, page_size, max_blocks;
    float scale_log2e;
    int window;
    int num_splits;
    int row_tiles;                 // row tiles per sequence the grid provides
    int q_filter;                  // 0: every sequence, 1: only q_len == 1, 2: only q_len > 1
};

template <int WARPS_M, int WARPS_N, int NSTAGES>
__global__ void __launch_bounds__(WARPS_M * WARPS_N * 32)
flash_paged_kernel(const FlashParams p) {
    rv_pdl_launch_dependents();
    // The step's metadata (sequence starts, context lengths, block tables) was copied to the device
    // before the step's first kernel started, so it is read here without waiting for the kernel
    // that precedes this one in the stream; q and the cache, which that kernel may still be
    // writing, are touched only after rv_pdl_wait() below.
    constexpr int HD = HEAD_DIM;
    constexpr int M_TILE = 16 * WARPS_M;
    constexpr int KW = KV_TILE / WARPS_N;          // keys of a tile that one warp owns
    constexpr int NTHREADS = WARPS_M * WARPS_N * 32;
    constexpr int CHUNKS = HD / 8;                 // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char smem[];

    const int seq = blockIdx.z, kvh = blockIdx.y;
    const int tile_m = blockIdx.x / p.num_splits, split = blockIdx.x - tile_m * p.num_splits;
    const int G = p.nh / p.nkv;
    const int ctx = p.ctx_lens[seq];
    const int q_start = p.cu_seqlens[seq];
    const int q_len = p.cu_seqlens[seq + 1] - q_start;
    const int rows_total = q_len * G;
    const int row0 = tile_m * M_TILE;
    if (q_len <= 0 || row0 >= rows_total || (p.q_filter == 1 && q_len != 1) || (p.q_filter == 2 && q_len == 1)) {
        rv_pdl_wait();          // a CTA without work still keeps the order of the chain of kernels
        return;
    }

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_m = warp / WARPS_N, warp_n = warp - warp_m * WARPS_N;
    const int quad = lane >> 2, tq = lane & 3;

    // the two rows this thread holds of its warp's 16
    int r[2], pos[2], lo[2], head[2], tok[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        r[i] = row0 + warp_m * 16 + quad + 8 * i;
        const bool in_range = r[i] < rows_total;
        const int t = in_range ? r[i] / G : 0;
        tok[i] = q_start + t;
        head[i] = kvh * G + (in_range ? r[i] - t * G : 0);
        valid[i] = in_range && ctx > 0;
        pos[i] = valid[i] ? ctx - q_len + t : -1;
        lo[i] = (p.window > 0 && pos[i] - p.window + 1 > 0) ? pos[i] - p.window + 1 : 0;
    }

    // key range of the whole row tile, and this split's share of its key tiles
    const int last_row = min(rows_total, row0 + M_TILE) - 1;
    const int pos_first = ctx - q_len + row0 / G, pos_last = ctx - q_len + last_row / G;
    const int key_lo = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    const int key_hi = ctx > 0 ? pos_last + 1 : 0;
    const int tile_lo = key_lo / KV_TILE, tile_hi = (key_hi + KV_TILE - 1) / KV_TILE;
    const int per_split = (tile_hi - tile_lo + p.num_splits - 1) / p.num_splits;
    const int t_begin = tile_lo + split * per_split;
    const int t_end = min(tile_hi, t_begin + per_split);

    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    const int* table = p.block_tables + (size_t)seq * p.max_blocks;
    // The page numbers of this CTA's key range are copied to shared memory once: a tile's loads
    // then start without first waiting for a read of the block table in global memory.
    __shared__ int s_table[TABLE_CACHE];
    const int blk_lo = (t_begin * KV_TILE) >> p.page_shift;
    const int blk_hi = t_begin < t_end ? ((min(t_end * KV_TILE, key_hi) - 1) >> p.page_shift) + 1 : blk_lo;
    const bool table_cached = blk_hi - blk_lo <= TABLE_CACHE;
    if (table_cached) {
        for (int i = tid; i < blk_hi - blk_lo; i += NTHREADS) s_table[i] = table[blk_lo + i];
        __syncthreads();
    }
    rv_pdl_wait();

    // Q fragments (A operand, 16 rows x HD), straight from global memory
    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const __nv_bfloat16* qp = p.q + ((size_t)tok[i] * p.nh + head[i]) * HD + ks * 16 + tq * 2;
            qa[ks][i] = valid[i] ? *reinterpret_cast<const uint32_t*>(qp) : 0u;
            qa[ks][i + 2] = valid[i] ? *reinterpret_cast<const uint32_t*>(qp + 8) : 0u;
        }
    }
    const size_t page_stride = (size_t)2 * p.nkv * p.page_size * HD;
    const size_t v_off = (size_t)p.nkv * p.page_size * HD;
    const __nv_bfloat16* kv_base = p.cache + (size_t)kvh * p.page_size * HD;

    auto load_tile = [&](int t, int stage) {
        unsigned char* ks = smem + (size_t)stage * 2 * TILE_BYTES;
        unsigned char* vs = ks + TILE_BYTES;
        for (int idx = tid; idx < KV_TILE * CHUNKS; idx += NTHREADS) {
            const int row = idx / CHUNKS, c = idx - row * CHUNKS;
            const int key = t * KV_TILE + row;
            const bool ok = key >= key_lo && key < key_hi;
            const __nv_bfloat16* src = p.cache;
            if (ok) {
                const int blk = key >> p.page_shift;
                const int page = table_cached ? s_table[blk - blk_lo] : table[blk];
                src = kv_base + (size_t)page * page_stride + (size_t)(key & (p.page_size - 1)) * HD + c * 8;
            }
            cp_async_16(ks + row * ROW_BYTES + c * 16, src, ok);
            cp_async_16(vs + row * ROW_BYTES + c * 16, ok ? src + v_off : src, ok);
        }
    };

    // NSTAGES - 1 tiles are requested ahead of the one being used
#pragma unroll
    for (int i = 0; i < NSTAGES - 1; ++i) {
        if (t_begin + i < t_end) load_tile(t_begin + i, i);
        cp_async_commit();
    }
    int stage = 0;
    for (int t = t_begin; t < t_end; ++t) {
        if (t + NSTAGES - 1 < t_end) load_tile(t + NSTAGES - 1, (stage + NSTAGES - 1) % NSTAGES);
        cp_async_commit();
        cp_async_wait<NSTAGES - 1>();
        __syncthreads();
        const unsigned char* ks = smem + (size_t)stage * 2 * TILE_BYTES;
        const unsigned char* vs = ks + TILE_BYTES;

        // S = Q K^T for this warp's rows and its KW keys of the tile
        float s[KW / 8][4];
#pragma unroll
        for (int n = 0; n < KW / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < KW / 16; ++n2) {
                uint32_t b[4];
                const int key_row = warp_n * KW + n2 * 16 + (lane >> 4) * 8 + (lane & 7);
                const int col = kk * 16 + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(b, ks + key_row * ROW_BYTES + col * 2);
                mma_bf16(s[2 * n2], qa[kk], b[0], b[1]);
                mma_bf16(s[2 * n2 + 1], qa[kk], b[2], b[3]);
            }
        }
        // scale, mask, running maximum
        const int key0 = t * KV_TILE + warp_n * KW + tq * 2;
        float m_tile[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < KW / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = e >> 1;
                const int key = key0 + n * 8 + (e & 1);
                const bool see = key <= pos[i] && key >= lo[i];
                const float v = see ? s[n][e] * p.scale_log2e : -INFINITY;
                s[n][e] = v;
                m_tile[i] = fmaxf(m_tile[i], v);
            }
        }
        float alpha[2], m_safe[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            m_tile[i] = fmaxf(m_tile[i], __shfl_xor_sync(0xffffffffu, m_tile[i], 1));
            m_tile[i] = fmaxf(m_tile[i], __shfl_xor_sync(0xffffffffu, m_tile[i], 2));
            const float m_new = fmaxf(m_run[i], m_tile[i]);
            m_safe[i] = m_new == -INFINITY ? 0.f : m_new;
            alpha[i] = exp2f(m_run[i] - m_safe[i]);
            m_run[i] = m_new;
        }
        float l_tile[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < KW / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = exp2f(s[n][e] - m_safe[e >> 1]);
                s[n][e] = pv;
                l_tile[e >> 1] += pv;
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * alpha[i] + l_tile[i];
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
            o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < KW / 16; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int n2 = 0; n2 < HD / 16; ++n2) {
                uint32_t b[4];
                const int key_row = warp_n * KW + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                const int col = n2 * 16 + (lane >> 4) * 8;
                ldmatrix_x4_trans(b, vs + key_row * ROW_BYTES + col * 2);
                mma_bf16(o[2 * n2], pa, b[0], b[1]);
                mma_bf16(o[2 * n2 + 1], pa, b[2], b[3]);
            }
        }
        __syncthreads();
        stage = (stage + 1) % NSTAGES;
    }
    cp_async_wait<0>();

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }

    if (WARPS_N > 1) {
        // Merge the warps that shared the rows: (m, l, O) of the real rows go to shared memory (the
        // key/value buffers are free now), then all threads of the CTA share the work of adding
        // them up, one output element at a time, and write the result.  WARPS_M is 1 here.
        __syncthreads();
        float* mo = reinterpret_cast<float*>(smem);                 // [WARPS_N][16][HD]
        float* mml = mo + WARPS_N * 16 * HD;                        // [WARPS_N][16][2]
        const int n_rows = min(16, rows_total - row0);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = quad + 8 * i;
            if (row >= n_rows) continue;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
                float* dst = mo + ((size_t)warp_n * 16 + row) * HD + n * 8 + tq * 2;
                dst[0] = o[n][2 * i]; dst[1] = o[n][2 * i + 1];
            }
            if (tq == 0) {
                mml[(warp_n * 16 + row) * 2] = m_run[i];
                mml[(warp_n * 16 + row) * 2 + 1] = l_run[i];
            }
        }
        __syncthreads();
        for (int idx = tid; idx < n_rows * HD; idx += NTHREADS) {
            const int row = idx / HD, d = idx - row * HD;
            float m_all = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS_N; ++w) m_all = fmaxf(m_all, mml[(w * 16 + row) * 2]);
            const float m_s = m_all == -INFINITY ? 0.f : m_all;
            float l_all = 0.f, acc = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS_N; ++w) {
                const float f = exp2f(mml[(w * 16 + row) * 2] - m_s);
                l_all += mml[(w * 16 + row) * 2 + 1] * f;
                acc += mo[((size_t)w * 16 + row) * HD + d] * f;
            }
            const int rr = row0 + row;
            const int t = rr / G;
            const size_t row_out = (size_t)(q_start + t) * p.nh + kvh * G + (rr - t * G);
            if (p.num_splits == 1) {
                p.out[row_out * HD + d] = __float2bfloat16_rn(acc * (l_all > 0.f ? 1.f / l_all : 0.f));
            } else {
                const size_t prow = (size_t)split * p.n_tokens * p.nh + row_out;
                p.part_o[prow * HD + d] = acc;
                if (d == 0) { p.part_ml[prow * 2] = m_all; p.part_ml[prow * 2 + 1] = l_all; }
            }
        }
        return;
    }

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (r[i] >= rows_total) continue;
        const size_t row_out = (size_t)tok[i] * p.nh + head[i];
        if (p.num_splits == 1) {
            const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
            __nv_bfloat16* dst = p.out + row_out * HD + tq * 2;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n)
                *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
        } else {
            const size_t prow = (size_t)split * p.n_tokens * p.nh + row_out;
            float* dst = p.part_o + prow * HD + tq * 2;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) { dst[n * 8] = o[n][2 * i]; dst[n * 8 + 1] = o[n][2 * i + 1]; }
            if (tq == 0) { p.part_ml[prow * 2] = m_run[i]; p.part_ml[prow * 2 + 1] = l_run[i]; }
        }
    }
}

// Element d of a row's attention output from the partial results of the key splits.  Eight splits
// are read at a time, maxima, denominators and sums together, so that the merge costs one round
// trip to L2 per eight splits; the running result is rescaled as in the attention kernel itself.
__device__ __forceinline__ float merge_splits(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              size_t row, size_t rows, int num_splits, int d) {
    float m_run = -INFINITY, l_run = 0.f, acc = 0.f;
    for (int s0 = 0; s0 < num_splits; s0 += 8) {
        float m[8], l[8], o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const bool have = s0 + i < num_splits;
            const size_t r = (size_t)(have ? s0 + i : s0) * rows + row;
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml) + r);
            m[i] = have ? ml.x : -INFINITY;
            l[i] = have ? ml.y : 0.f;
            o[i] = __ldcg(part_o + r * HEAD_DIM + d);
        }
        float m_new = m_run;
#pragma unroll
        for (int i = 0; i < 8; ++i) m_new = fmaxf(m_new, m[i]);
        const float m_s = m_new == -INFINITY ? 0.f : m_new;
        const float keep = exp2f(m_run - m_s);          // 0 while nothing has been seen
        l_run *= keep;
        acc *= keep;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float f = exp2f(m[i] - m_s);           // 0 for an empty or absent split
            l_run += l[i] * f;
            if (f > 0.f) acc += o[i] * f;                // an empty split's sum may hold anything
        }
        m_run = m_new;
    }
    return acc * (l_run > 0.f ? 1.f / l_run : 0.f);
}

// The same for four neighbouring elements d .. d + 3 (d a multiple of 4), every split's loads in flight together.
__device__ __forceinline__ float4 merge_splits4(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                size_t row, size_t rows, int num_splits, int d) {
    float m_run = -INFINITY, l_run = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < num_splits; s0 += 8) {
        float m[8], l[8];
        float4 o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const bool have = s0 + i < num_splits;
            const size_t r = (size_t)(have ? s0 + i : s0) * rows + row;
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml) + r);
            m[i] = have ? ml.x : -INFINITY;
            l[i] = have ? ml.y : 0.f;
            o[i] = __ldcg(reinterpret_cast<const float4*>(part_o + r * HEAD_DIM + d));
        }
        float m_new = m_run;
#pragma unroll
        for (int i = 0; i < 8; ++i) m_new = fmaxf(m_new, m[i]);
        const float m_s = m_new == -INFINITY ? 0.f : m_new;
        const float keep = exp2f(m_run - m_s);          // 0 while nothing has been seen
        l_run *= keep;
        acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float f = exp2f(m[i] - m_s);           // 0 for an empty or absent split
            l_run += l[i] * f;
            if (f > 0.f) { acc.x += o[i].x * f; acc.y += o[i].y * f; acc.z += o[i].z * f; acc.w += o[i].w * f; }
        }
        m_run = m_new;
    }
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    return make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
}

// Merge the partial results of the key splits: HEAD_DIM / 4 threads per (token, head) row, four neighbouring
// elements each (16-byte reads of the partials, an 8-byte store); a block of 128 threads takes several rows.
#define COMBINE_TPR (HEAD_DIM / 4)                 // threads per row
#define COMBINE_ROWS (128 / COMBINE_TPR)           // rows per block
__global__ void flash_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                     __nv_bfloat16* __restrict__ out, int rows, int num_splits) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int r = threadIdx.x / COMBINE_TPR, d = (threadIdx.x - r * COMBINE_TPR) * 4;
    const int row = blockIdx.x * COMBINE_ROWS + r;
    if (r >= COMBINE_ROWS || row >= rows) return;
    const float4 v = merge_splits4(part_o, part_ml, (size_t)row, (size_t)rows, num_splits, d);
    uint2 o2;
    o2.x = pack_bf16(v.x, v.y);
    o2.y = pack_bf16(v.z, v.w);
    *reinterpret_cast<uint2*>(out + (size_t)row * HEAD_DIM + d) = o2;
}

// ---------------------------------------------------------------------------------------------
// Decode attention fed by TMA (head sizes 64 and 128, pages of at least 8 keys).  The decode tiling
// of the kernel above - 16 rows, four warps that own 16 of a tile's 64 keys each, key splits over
// CTAs, the same arithmetic in the same order, so the same bits - but the tiles are brought in by
// a fifth warp with cp.async.bulk.tensor, one box per (page, 64 elements of the head) through the
// block table, into 128-byte-swizzled stages that mbarriers hand back and forth:
//   full[stage]   the producer's expect_tx + the boxes' bytes        -> the four consumer warps
//   empty[stage]  one arrival per consumer warp after its last read  -> the producer
// The consumer warps issue no address arithmetic or copy instructions at all.  Only the box that
// holds the sequence's newest key (written by the kernel before this one) has to wait for that
// kernel; with `early` set, the producer requests all older keys before griddepcontrol.wait, so
// that they arrive while the predecessor's last CTAs drain.
// A CTA never returns while one of its copies is in flight: every box that is requested is waited
// for by the consumers, and after a wait that gave up (bounded, with a status word) the producer
// waits, again bounded, for what it has requested - shared memory that a later CTA of the grid
// inherits is never written by a copy of an earlier one.
#if HEAD_DIM == 64 || HEAD_DIM == 128
#define RV_HAVE_TMA_DECODE 1
#include "tcgen05.cuh"
#define TMA_HALVES (HEAD_DIM / 64)
#define TMA_SLAB (KV_TILE * 128)                    // one 64-element slab of a tile: 64 keys x 128 bytes
#define TMA_TILE_BYTES (TMA_HALVES * TMA_SLAB)      // K (or V) of a 64-key tile
#ifndef TMA_STAGES
#define TMA_STAGES 2
#endif
#define TMA_THREADS 160                             // 4 consumer warps + 1 producer warp
#ifndef TMA_MIN_CTAS
#define TMA_MIN_CTAS 3                              // CTAs per SM the register budget is held to
#endif

// byte offset of element `col` of key `row` inside a tile of 128-byte-swizzled slabs
__device__ __forceinline__ int tma_swz(int row, int col) {
    return (col >> 6) * TMA_SLAB + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4);
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int NST>
__global__ void __launch_bounds__(TMA_THREADS, TMA_MIN_CTAS)
flash_decode_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const FlashParams p, int* status, int early) {
    rv_pdl_launch_dependents();
    constexpr int HD = HEAD_DIM;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* k_s = smem;                                   // [NST][TMA_TILE_BYTES]
    unsigned char* v_s = smem + NST * TMA_TILE_BYTES;            // [NST][TMA_TILE_BYTES]
    __shared__ __align__(8) uint64_t bars[2 * NST];
    __shared__ volatile int abort_flag;

    const int seq = blockIdx.z, kvh = blockIdx.y;
    const int tile_m = blockIdx.x / p.num_splits, split = blockIdx.x - tile_m * p.num_splits;
    const int G = p.nh / p.nkv;
    const int ctx = p.ctx_lens[seq];
    const int q_start = p.cu_seqlens[seq];
    const int q_len = p.cu_seqlens[seq + 1] - q_start;
    const int rows_total = q_len * G;
    const int row0 = tile_m * 16;
    if (q_len <= 0 || row0 >= rows_total || (p.q_filter == 1 && q_len != 1) || (p.q_filter == 2 && q_len == 1)) {
        rv_pdl_wait();
        return;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[NST]);

    // key range of the row tile and this split's share of its key tiles (as in the kernel above)
    const int last_row = min(rows_total, row0 + 16) - 1;
    const int pos_first = ctx - q_len + row0 / G, pos_last = ctx - q_len + last_row / G;
    const int key_lo = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    const int key_hi = ctx > 0 ? pos_last + 1 : 0;
    const int tile_lo = key_lo / KV_TILE, tile_hi = (key_hi + KV_TILE - 1) / KV_TILE;
    const int per_split = (tile_hi - tile_lo + p.num_splits - 1) / p.num_splits;
    const int t_begin = tile_lo + split * per_split;
    const int t_end = min(tile_hi, t_begin + per_split);
    const int n_tiles = t_end > t_begin ? t_end - t_begin : 0;

    if (tid == 0) {
        tma_prefetch_descriptor(&map_kv);
        abort_flag = 0;
#pragma unroll
        for (int s = 0; s < NST; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // value stages start as zeros: keys of a tile that are not requested (beyond the context, or
    // below a window) meet a probability of zero, which must not find a NaN left in shared memory
    for (int i = tid; i < NST * TMA_TILE_BYTES / 16; i += TMA_THREADS) reinterpret_cast<uint4*>(v_s)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    if (warp == 4) {
        // ------------------------------------------------------------ producer warp
        const int* table = p.block_tables + (size_t)seq * p.max_blocks;
        const int box_keys = p.page_size < KV_TILE ? p.page_size : KV_TILE;
        const int boxes = KV_TILE / box_keys;
        bool waited = false;
        if (!early) { rv_pdl_wait(); waited = true; }
        int issued = 0;
        bool ok = true;
        for (int i = 0; i < n_tiles && ok; ++i) {
            const int t = t_begin + i, stage = i % NST, use = i / NST;
            if (use > 0) {
                int ok_l = 1;
                if (lane == 0) ok_l = mbar_wait(empty0 + 8 * stage, (use - 1) & 1, &abort_flag, 1) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok_l, 0) != 0;
                if (!ok) break;
            }
            // the newest key of the sequence was written by the kernel before this one
            if (!waited && (t + 1) * KV_TILE >= ctx) { rv_pdl_wait(); waited = true; }
            const int key = t * KV_TILE + lane * box_keys;
            int page = -1;
            if (lane < boxes && key < key_hi && key + box_keys > key_lo) page = __ldg(table + (key >> p.page_shift));
            const unsigned mask = __ballot_sync(0xffffffffu, page >= 0);
            const uint32_t bar = full0 + 8 * stage;
            if (lane == 0) mbar_expect_tx(bar, (uint32_t)__popc(mask) * 2u * TMA_HALVES * (uint32_t)box_keys * 128u);
            __syncwarp();
            if (page >= 0) {
                const int row_k = ((page * 2) * p.nkv + kvh) * p.page_size + (key & (p.page_size - 1));
                const int row_v = row_k + p.nkv * p.page_size;
                const uint32_t dk = smem_u32(k_s) + (uint32_t)stage * TMA_TILE_BYTES + (uint32_t)lane * box_keys * 128;
                const uint32_t dv = smem_u32(v_s) + (uint32_t)stage * TMA_TILE_BYTES + (uint32_t)lane * box_keys * 128;
#pragma unroll
                for (int h = 0; h < TMA_HALVES; ++h) {
                    tma_load_2d(dk + h * TMA_SLAB, &map_kv, h * 64, row_k, bar);
                    tma_load_2d(dv + h * TMA_SLAB, &map_kv, h * 64, row_v, bar);
                }
            }
            __syncwarp();
            ++issued;
        }
        if (!waited) rv_pdl_wait();
        if (!ok || abort_flag != 0) {
            // something gave up: wait (bounded) for the copies still in flight before this CTA's shared memory is given up
            if (lane == 0) {
                volatile int ignore = 0;
                for (int i = max(0, issued - NST); i < issued; ++i)
                    mbar_wait(full0 + 8 * (i % NST), (i / NST) & 1, &ignore, 0);
            }
        }
    } else {
        // ------------------------------------------------------------ consumer warps
        const int warp_n = warp;
        const int quad = lane >> 2, tq = lane & 3;
        int r[2], pos[2], lo[2], head[2], tok[2];
        bool valid[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            r[i] = row0 + quad + 8 * i;
            const bool in_range = r[i] < rows_total;
            const int t = in_range ? r[i] / G : 0;
            tok[i] = q_start + t;
            head[i] = kvh * G + (in_range ? r[i] - t * G : 0);
            valid[i] = in_range && ctx > 0;
            pos[i] = valid[i] ? ctx - q_len + t : -1;
            lo[i] = (p.window > 0 && pos[i] - p.window + 1 > 0) ? pos[i] - p.window + 1 : 0;
        }
        float o[HD / 8][4];
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
        rv_pdl_wait();
        uint32_t qa[HD / 16][4];
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const __nv_bfloat16* qp = p.q + ((size_t)tok[i] * p.nh + head[i]) * HD + ks * 16 + tq * 2;
                qa[ks][i] = valid[i] ? *reinterpret_cast<const uint32_t*>(qp) : 0u;
                qa[ks][i + 2] = valid[i] ? *reinterpret_cast<const uint32_t*>(qp + 8) : 0u;
            }
        }
        bool ok = true;
        for (int it = 0; it < n_tiles; ++it) {
            const int t = t_begin + it, stage = it % NST;
            if (!mbar_wait(full0 + 8 * stage, (it / NST) & 1, &abort_flag, 2)) { ok = false; break; }
            const unsigned char* ks = k_s + (size_t)stage * TMA_TILE_BYTES;
            const unsigned char* vs = v_s + (size_t)stage * TMA_TILE_BYTES;
            // S = Q K^T for the rows and this warp's 16 keys of the tile
            float s[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                uint32_t b[4];
                const int key_row = warp_n * 16 + (lane >> 4) * 8 + (lane & 7);
                const int col = kk * 16 + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(b, ks + tma_swz(key_row, col));
                mma_bf16(s[0], qa[kk], b[0], b[1]);
                mma_bf16(s[1], qa[kk], b[2], b[3]);
            }
            const int key0 = t * KV_TILE + warp_n * 16 + tq * 2;
            float m_tile[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < 2; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const int key = key0 + n * 8 + (e & 1);
                    const bool see = key <= pos[i] && key >= lo[i];
                    const float v = see ? s[n][e] * p.scale_log2e : -INFINITY;
                    s[n][e] = v;
                    m_tile[i] = fmaxf(m_tile[i], v);
                }
            }
            float alpha[2], m_safe[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                m_tile[i] = fmaxf(m_tile[i], __shfl_xor_sync(0xffffffffu, m_tile[i], 1));
                m_tile[i] = fmaxf(m_tile[i], __shfl_xor_sync(0xffffffffu, m_tile[i], 2));
                const float m_new = fmaxf(m_run[i], m_tile[i]);
                m_safe[i] = m_new == -INFINITY ? 0.f : m_new;
                alpha[i] = exp2f(m_run[i] - m_safe[i]);
                m_run[i] = m_new;
            }
            float l_tile[2] = {0.f, 0.f};
#pragma unroll
            for (int n = 0; n < 2; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = exp2f(s[n][e] - m_safe[e >> 1]);
                    s[n][e] = pv;
                    l_tile[e >> 1] += pv;
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * alpha[i] + l_tile[i];
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
                o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
                o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
            }
            // O += P V
            uint32_t pa[4];
            pa[0] = pack_bf16(s[0][0], s[0][1]);
            pa[1] = pack_bf16(s[0][2], s[0][3]);
            pa[2] = pack_bf16(s[1][0], s[1][1]);
            pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
            for (int n2 = 0; n2 < HD / 16; ++n2) {
                uint32_t b[4];
                const int key_row = warp_n * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                const int col = n2 * 16 + (lane >> 4) * 8;
                ldmatrix_x4_trans(b, vs + tma_swz(key_row, col));
                mma_bf16(o[2 * n2], pa, b[0], b[1]);
                mma_bf16(o[2 * n2 + 1], pa, b[2], b[3]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * stage);      // this warp has read the stage for the last time
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
            l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
        }
        // merge the four warps through shared memory (every requested tile has arrived and been read:
        // no copy is in flight, the stages are free) - unless a wait gave up: then nothing is written
        consumer_sync();
        if (abort_flag == 0 && ok) {
            float* mo = reinterpret_cast<float*>(smem);                 // [4][16][HD]
            float* mml = mo + 4 * 16 * HD;                              // [4][16][2]
            const int n_rows = min(16, rows_total - row0);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int row = quad + 8 * i;
                if (row >= n_rows) continue;
#pragma unroll
                for (int n = 0; n < HD / 8; ++n) {
                    float* dst = mo + ((size_t)warp_n * 16 + row) * HD + n * 8 + tq * 2;
                    dst[0] = o[n][2 * i]; dst[1] = o[n][2 * i + 1];
                }
                if (tq == 0) {
                    mml[(warp_n * 16 + row) * 2] = m_run[i];
                    mml[(warp_n * 16 + row) * 2 + 1] = l_run[i];
                }
            }
            consumer_sync();
            for (int idx = tid; idx < n_rows * HD; idx += 128) {
                const int row = idx / HD, d = idx - row * HD;
                float m_all = -INFINITY;
#pragma unroll
                for (int w = 0; w < 4; ++w) m_all = fmaxf(m_all, mml[(w * 16 + row) * 2]);
                const float m_s = m_all == -INFINITY ? 0.f : m_all;
                float l_all = 0.f, acc = 0.f;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float f = exp2f(mml[(w * 16 + row) * 2] - m_s);
                    l_all += mml[(w * 16 + row) * 2 + 1] * f;
                    acc += mo[((size_t)w * 16 + row) * HD + d] * f;
                }
                const int rr = row0 + row;
                const int t = rr / G;
                const size_t row_out = (size_t)(q_start + t) * p.nh + kvh * G + (rr - t * G);
                if (p.num_splits == 1) {
                    p.out[row_out * HD + d] = __float2bfloat16_rn(acc * (l_all > 0.f ? 1.f / l_all : 0.f));
                } else {
                    const size_t prow = (size_t)split * p.n_tokens * p.nh + row_out;
                    p.part_o[prow * HD + d] = acc;
                    if (d == 0) { p.part_ml[prow * 2] = m_all; p.part_ml[prow * 2 + 1] = l_all; }
                }
            }
        }
    }
    __syncthreads();
    if (tid == 0 && abort_flag != 0 && status) atomicCAS(status, 0, abort_flag);
}
#endif   // HEAD_DIM 64 / 128

// ---------------------------------------------------------------------------------------------
// Decode attention with the work cut evenly: one token per sequence, as the decode tiling above,
// but the grid is a fixed number of CTAs (as many as stay resident: three per SM) and every CTA
// takes the same number of 64-key tiles.  The tiles of all (sequence, kv head) pairs form one list,
// sequence-major; CTA c takes the tiles [c W, (c + 1) W), W = ceil(total / CTAs), which is a run of
// pieces, each a range of tiles of one pair.  So no wave is left half empty and a CTA's fixed cost
// (about 4 us in the kernel above) is paid once or twice per CTA, not once per split.  Every piece
// leaves (unnormalised sum, maximum, denominator) in scratch memory at [piece of its pair]; the
// merge kernel below adds a pair's pieces, whose number the attention kernel writes per pair.
#define BAL_MAX_SEQS 256      // sequences per step this kernel serves (their tile counts live in shared memory)
#define BAL_TABLE_CACHE 512   // block-table entries of a piece kept in shared memory

struct BalancedParams {
    const __nv_bfloat16* q;        // [n_tokens, nh, HEAD_DIM]
    const __nv_bfloat16* cache;
    const int* block_tables;       // [num_seqs, max_blocks]
    const int* cu_seqlens;
    const int* ctx_lens;
    __nv_bfloat16* out;
    float* part_o;                 // [max_pieces, n_tokens * nh, HEAD_DIM]
    float* part_ml;                // [max_pieces, n_tokens * nh, 2]
    int* piece_count;              // [num_seqs * nkv]: pieces of each pair, written by the kernel
    int n_tokens, num_seqs, nh, nkv, page_shift, page_size, max_blocks, max_pieces;
    float scale_log2e;
    int window;
};

template <int NSTAGES>
__global__ void __launch_bounds__(128)
flash_decode_balanced_kernel(const BalancedParams p) {
    rv_pdl_launch_dependents();
    constexpr int HD = HEAD_DIM;
    constexpr int WARPS_N = 4, KW = KV_TILE / WARPS_N, NTHREADS = 128, CHUNKS = HD / 8;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_first[BAL_MAX_SEQS + 1];          // tiles of the sequences before this one
    __shared__ int s_lo[BAL_MAX_SEQS];                 // first key tile of the sequence (window)
    __shared__ int s_table[BAL_TABLE_CACHE];
    const int tid = threadIdx.x, lane = tid & 31, warp_n = tid >> 5;
    const int quad = lane >> 2, tq = lane & 3;
    const int G = p.nh / p.nkv;

    // ---- the list of tiles (step metadata: read before the wait for the previous kernel)
    for (int s = tid; s < p.num_seqs; s += NTHREADS) {
        const int ctx = p.ctx_lens[s];
        const int q_len = p.cu_seqlens[s + 1] - p.cu_seqlens[s];
        int lo = 0, n = 0;
        if (q_len == 1 && ctx > 0) {
            const int pos = ctx - 1;
            const int key_lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
            lo = key_lo / KV_TILE;
            n = (ctx + KV_TILE - 1) / KV_TILE - lo;
        }
        s_lo[s] = lo;
        s_first[s + 1] = n;
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        s_first[0] = 0;
        for (int s = 0; s < p.num_seqs; ++s) { run += s_first[s + 1]; s_first[s + 1] = run; }
    }
    __syncthreads();
    const int total = s_first[p.num_seqs] * p.nkv;
    const int ctas = gridDim.x, cta = blockIdx.x;
    const int W = total > 0 ? (total + ctas - 1) / ctas : 1;
    int u = cta * W;
    const int u_end = min(total, u + W);
    // Nothing is written before this wait: the buffers of this launch may be memory that a kernel
    // still running ahead of it in the stream uses under another name (a stream-ordered allocator
    // hands freed blocks out again at once).
    rv_pdl_wait();          // every CTA, with or without work, keeps the order of the chain of kernels
    // pieces of every pair, for the merge kernel: each CTA writes its share of the pairs
    for (int pair = cta * NTHREADS + tid; pair < p.num_seqs * p.nkv; pair += ctas * NTHREADS) {
        const int s = pair / p.nkv, kvh = pair - s * p.nkv;
        const int n = s_first[s + 1] - s_first[s];
        int count = 0;
        if (n > 0) {
            const int u_pair = s_first[s] * p.nkv + kvh * n;
            count = (u_pair + n - 1) / W - u_pair / W + 1;
        }
        p.piece_count[pair] = count;
    }
    if (u >= u_end) return;

    const size_t page_stride = (size_t)2 * p.nkv * p.page_size * HD;
    const size_t v_off = (size_t)p.nkv * p.page_size * HD;
    const size_t rows_all = (size_t)p.n_tokens * p.nh;

    // first sequence of the run: the last one whose tiles start at or before u
    int seq;
    {
        int lo = 0, hi = p.num_seqs - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_first[mid] * p.nkv <= u) lo = mid; else hi = mid - 1;
        }
        seq = lo;
    }
    while (u < u_end) {
        while (s_first[seq + 1] * p.nkv <= u) ++seq;                    // skips sequences without tiles
        const int n_seq = s_first[seq + 1] - s_first[seq];
        const int in_seq = u - s_first[seq] * p.nkv;
        const int kvh = in_seq / n_seq;
        const int t_rel = in_seq - kvh * n_seq;
        const int n_here = min(n_seq - t_rel, u_end - u);              // tiles of this piece
        const int u_pair = u - t_rel;
        const int piece = u / W - u_pair / W;                           // its place among the pair's pieces
        const int ctx = p.ctx_lens[seq];
        const int pos = ctx - 1;
        const int key_lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
        const int t_begin = s_lo[seq] + t_rel, t_end = t_begin + n_here;
        const int tok = p.cu_seqlens[seq];

        // rows quad and quad + 8 of the 16-row tile; only rows < G are query heads
        bool valid[2];
        int head[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = quad + 8 * i;
            valid[i] = r < G;
            head[i] = kvh * G + (r < G ? r : 0);
        }
        uint32_t qa[HD / 16][4];
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const __nv_bfloat16* qp = p.q + ((size_t)tok * p.nh + head[i]) * HD + ks * 16 + tq * 2;
                qa[ks][i] = valid[i] ? *reinterpret_cast<const uint32_t*>(qp) : 0u;
                qa[ks][i + 2] = valid[i] ? *reinterpret_cast<const uint32_t*>(qp + 8) : 0u;
            }
        }
        float o[HD / 8][4];
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

        const int* table = p.block_tables + (size_t)seq * p.max_blocks;
        const int blk_lo = (t_begin * KV_TILE) >> p.page_shift;
        const int blk_hi = ((min(t_end * KV_TILE, ctx) - 1) >> p.page_shift) + 1;
        const bool table_cached = blk_hi - blk_lo <= BAL_TABLE_CACHE;
        if (table_cached)
            for (int i = tid; i < blk_hi - blk_lo; i += NTHREADS) s_table[i] = table[blk_lo + i];
        __syncthreads();              // also: the merge of the piece before this one has left the buffers
        const __nv_bfloat16* kv_base = p.cache + (size_t)kvh * p.page_size * HD;

        auto load_tile = [&](int t, int stage) {
            unsigned char* ks = smem + (size_t)stage * 2 * TILE_BYTES;
            unsigned char* vs = ks + TILE_BYTES;
            for (int idx = tid; idx < KV_TILE * CHUNKS; idx += NTHREADS) {
                const int row = idx / CHUNKS, c = idx - row * CHUNKS;
                const int key = t * KV_TILE + row;
                const bool ok = key >= key_lo && key < ctx;
                const __nv_bfloat16* src = p.cache;
                if (ok) {
                    const int blk = key >> p.page_shift;
                    const int page = table_cached ? s_table[blk - blk_lo] : table[blk];
                    src = kv_base + (size_t)page * page_stride + (size_t)(key & (p.page_size - 1)) * HD + c * 8;
                }
                cp_async_16(ks + row * ROW_BYTES + c * 16, src, ok);
                cp_async_16(vs + row * ROW_BYTES + c * 16, ok ? src + v_off : src, ok);
            }
        };
#pragma unroll
        for (int i = 0; i < NSTAGES - 1; ++i) {
            if (t_begin + i < t_end) load_tile(t_begin + i, i);
            cp_async_commit();
        }
        int stage = 0;
        for (int t = t_begin; t < t_end; ++t) {
            if (t + NSTAGES - 1 < t_end) load_tile(t + NSTAGES - 1, (stage + NSTAGES - 1) % NSTAGES);
            cp_async_commit();
            cp_async_wait<NSTAGES - 1>();
            __syncthreads();
            const unsigned char* ks = smem + (size_t)stage * 2 * TILE_BYTES;
            const unsigned char* vs = ks + TILE_BYTES;
            float s[KW / 8][4];
#pragma unroll
            for (int n = 0; n < KW / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
                for (int n2 = 0; n2 < KW / 16; ++n2) {
                    uint32_t b[4];
                    const int key_row = warp_n * KW + n2 * 16 + (lane >> 4) * 8 + (lane & 7);
                    const int col = kk * 16 + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(b, ks + key_row * ROW_BYTES + col * 2);
                    mma_bf16(s[2 * n2], qa[kk], b[0], b[1]);
                    mma_bf16(s[2 * n2 + 1], qa[kk], b[2], b[3]);
                }
            }
            const int key0 = t * KV_TILE + warp_n * KW + tq * 2;
            float m_tile[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < KW / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + n * 8 + (e & 1);
                    const bool see = key <= pos && key >= key_lo;
                    const float v = see ? s[n][e] * p.scale_log2e : -INFINITY;
                    s[n][e] = v;
                    m_tile[e >> 1] = fmaxf(m_tile[e >> 1], v);
                }
            }
            float alpha[2], m_safe[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                m_tile[i] = fmaxf(m_tile[i], __shfl_xor_sync(0xffffffffu, m_tile[i], 1));
                m_tile[i] = fmaxf(m_tile[i], __shfl_xor_sync(0xffffffffu, m_tile[i], 2));
                const float m_new = fmaxf(m_run[i], m_tile[i]);
                m_safe[i] = m_new == -INFINITY ? 0.f : m_new;
                alpha[i] = exp2f(m_run[i] - m_safe[i]);
                m_run[i] = m_new;
            }
            float l_tile[2] = {0.f, 0.f};
#pragma unroll
            for (int n = 0; n < KW / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = exp2f(s[n][e] - m_safe[e >> 1]);
                    s[n][e] = pv;
                    l_tile[e >> 1] += pv;
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * alpha[i] + l_tile[i];
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
                o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
                o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
            }
#pragma unroll
            for (int kk = 0; kk < KW / 16; ++kk) {
                uint32_t pa[4];
                pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int n2 = 0; n2 < HD / 16; ++n2) {
                    uint32_t b[4];
                    const int key_row = warp_n * KW + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                    const int col = n2 * 16 + (lane >> 4) * 8;
                    ldmatrix_x4_trans(b, vs + key_row * ROW_BYTES + col * 2);
                    mma_bf16(o[2 * n2], pa, b[0], b[1]);
                    mma_bf16(o[2 * n2 + 1], pa, b[2], b[3]);
                }
            }
            __syncthreads();
            stage = (stage + 1) % NSTAGES;
        }
        cp_async_wait<0>();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
            l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
        }
        // ---- merge the four warps through shared memory and write the piece's partial result
        __syncthreads();
        float* mo = reinterpret_cast<float*>(smem);                 // [WARPS_N][16][HD]
        float* mml = mo + WARPS_N * 16 * HD;                        // [WARPS_N][16][2]
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = quad + 8 * i;
            if (row >= G) continue;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
                float* dst = mo + ((size_t)warp_n * 16 + row) * HD + n * 8 + tq * 2;
                dst[0] = o[n][2 * i]; dst[1] = o[n][2 * i + 1];
            }
            if (tq == 0) {
                mml[(warp_n * 16 + row) * 2] = m_run[i];
                mml[(warp_n * 16 + row) * 2 + 1] = l_run[i];
            }
        }
        __syncthreads();
        for (int idx = tid; idx < G * HD; idx += NTHREADS) {
            const int row = idx / HD, d = idx - row * HD;
            float m_all = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS_N; ++w) m_all = fmaxf(m_all, mml[(w * 16 + row) * 2]);
            const float m_s = m_all == -INFINITY ? 0.f : m_all;
            float l_all = 0.f, acc = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS_N; ++w) {
                const float f = exp2f(mml[(w * 16 + row) * 2] - m_s);
                l_all += mml[(w * 16 + row) * 2 + 1] * f;
                acc += mo[((size_t)w * 16 + row) * HD + d] * f;
            }
            const size_t prow = (size_t)piece * rows_all + (size_t)tok * p.nh + kvh * G + row;
            p.part_o[prow * HD + d] = acc;
            if (d == 0) { p.part_ml[prow * 2] = m_all; p.part_ml[prow * 2 + 1] = l_all; }
        }
        u += n_here;
    }
}

#ifdef RV_HAVE_TMA_DECODE
// The evenly cut kernel fed by TMA: the tile list, the pieces and the arithmetic of the kernel above (so the same
// bits), the tiles brought by a fifth warp as in flash_decode_tma_kernel.  The producer walks the CTA's run of
// tiles on its own, across the pieces' borders: while the four consumer warps merge a piece and load the next
// piece's queries, the next piece's first tiles are already on their way.  The merge buffer lies behind the ring
// (the ring is never idle), sized for the group's rows.
// Sequences per step: with 240 the kernel's static shared memory stays within 1 KB, and three CTAs (two stages of
// keys and values, the merge buffer of a group of four heads) just fit an SM.
#define BAL_TMA_MAX_SEQS 240
template <int NST>
__global__ void __launch_bounds__(TMA_THREADS, TMA_MIN_CTAS)
flash_decode_balanced_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const BalancedParams p, int* status) {
    rv_pdl_launch_dependents();
    constexpr int HD = HEAD_DIM;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* k_s = smem;                                   // [NST][TMA_TILE_BYTES]
    unsigned char* v_s = smem + NST * TMA_TILE_BYTES;            // [NST][TMA_TILE_BYTES]
    float* mo = reinterpret_cast<float*>(smem + 2 * NST * TMA_TILE_BYTES);       // [4 warps][G][HD], then [4][G][2]
    __shared__ __align__(8) uint64_t bars[2 * NST];
    __shared__ volatile int abort_flag;
    __shared__ int s_first[BAL_TMA_MAX_SEQS + 1];      // tiles of the sequences before this one (a sequence's first key
                                                       // tile under a window is worked out again where it is needed)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int quad = lane >> 2, tq = lane & 3;
    const int G = p.nh / p.nkv;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[NST]);

    // ---- the list of tiles (step metadata: read before the wait for the previous kernel)
    for (int s = tid; s < p.num_seqs; s += TMA_THREADS) {
        const int ctx = p.ctx_lens[s];
        const int q_len = p.cu_seqlens[s + 1] - p.cu_seqlens[s];
        int lo = 0, n = 0;
        if (q_len == 1 && ctx > 0) {
            const int pos = ctx - 1;
            const int key_lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
            lo = key_lo / KV_TILE;
            n = (ctx + KV_TILE - 1) / KV_TILE - lo;
        }
        s_first[s + 1] = n;
    }
    if (tid == 0) {
        tma_prefetch_descriptor(&map_kv);
        abort_flag = 0;
#pragma unroll
        for (int s = 0; s < NST; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // value stages start as zeros (keys of a tile that are not requested meet a probability of zero)
    for (int i = tid; i < NST * TMA_TILE_BYTES / 16; i += TMA_THREADS) reinterpret_cast<uint4*>(v_s)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        s_first[0] = 0;
        for (int s = 0; s < p.num_seqs; ++s) { run += s_first[s + 1]; s_first[s + 1] = run; }
    }
    __syncthreads();
    const int total = s_first[p.num_seqs] * p.nkv;
    const int ctas = gridDim.x, cta = blockIdx.x;
    const int W = total > 0 ? (total + ctas - 1) / ctas : 1;
    const int u0 = cta * W;
    const int u_end = min(total, u0 + W);
    // first sequence of the run: the last one whose tiles start at or before u0 (both roles walk on from it)
    int seq0 = 0;
    if (u0 < u_end) {
        int lo = 0, hi = p.num_seqs - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_first[mid] * p.nkv <= u0) lo = mid; else hi = mid - 1;
        }
        seq0 = lo;
    }

    if (warp == 4) {
        // ------------------------------------------------------------ producer warp
        const int box_keys = p.page_size < KV_TILE ? p.page_size : KV_TILE;
        const int boxes = KV_TILE / box_keys;
        bool waited = false, ok = true;
        int issued = 0, seq = seq0;
        for (int u = u0; u < u_end && ok; ++u, ++issued) {
            while (s_first[seq + 1] * p.nkv <= u) ++seq;
            const int n_seq = s_first[seq + 1] - s_first[seq];
            const int in_seq = u - s_first[seq] * p.nkv;
            const int kvh = in_seq / n_seq;
            const int stage = issued % NST, use = issued / NST;
            if (use > 0) {
                int ok_l = 1;
                if (lane == 0) ok_l = mbar_wait(empty0 + 8 * stage, (use - 1) & 1, &abort_flag, 1) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok_l, 0) != 0;
                if (!ok) break;
            }
            const int ctx = p.ctx_lens[seq];
            const int key_lo = (p.window > 0 && ctx - p.window > 0) ? ctx - p.window : 0;
            const int t = key_lo / KV_TILE + (in_seq - kvh * n_seq);
            // the newest key of a sequence was written by the kernel before this one
            if (!waited && (t + 1) * KV_TILE >= ctx) { rv_pdl_wait(); waited = true; }
            const int* table = p.block_tables + (size_t)seq * p.max_blocks;
            const int key = t * KV_TILE + lane * box_keys;
            int page = -1;
            if (lane < boxes && key < ctx && key + box_keys > key_lo) page = __ldg(table + (key >> p.page_shift));
            const unsigned mask = __ballot_sync(0xffffffffu, page >= 0);
            const uint32_t bar = full0 + 8 * stage;
            if (lane == 0) mbar_expect_tx(bar, (uint32_t)__popc(mask) * 2u * TMA_HALVES * (uint32_t)box_keys * 128u);
            __syncwarp();
            if (page >= 0) {
                const int row_k = ((page * 2) * p.nkv + kvh) * p.page_size + (key & (p.page_size - 1));
                const int row_v = row_k + p.nkv * p.page_size;
                const uint32_t dk = smem_u32(k_s) + (uint32_t)stage * TMA_TILE_BYTES + (uint32_t)lane * box_keys * 128;
                const uint32_t dv = smem_u32(v_s) + (uint32_t)stage * TMA_TILE_BYTES + (uint32_t)lane * box_keys * 128;
#pragma unroll
                for (int h = 0; h < TMA_HALVES; ++h) {
                    tma_load_2d(dk + h * TMA_SLAB, &map_kv, h * 64, row_k, bar);
                    tma_load_2d(dv + h * TMA_SLAB, &map_kv, h * 64, row_v, bar);
                }
            }
            __syncwarp();
        }
        if (!waited) rv_pdl_wait();
        if (!ok || abort_flag != 0) {
            // something gave up: wait (bounded) for the copies still in flight before this CTA's shared memory is given up
            if (lane == 0) {
                volatile int ignore = 0;
                for (int i = max(0, issued - NST); i < issued; ++i)
                    mbar_wait(full0 + 8 * (i % NST), (i / NST) & 1, &ignore, 0);
            }
        }
    } else {
        // ------------------------------------------------------------ consumer warps
        const int warp_n = warp;
        // Nothing is written before this wait (see the kernel above).
        rv_pdl_wait();
        for (int pair = cta * 128 + tid; pair < p.num_seqs * p.nkv; pair += ctas * 128) {
            const int s = pair / p.nkv, kvh = pair - s * p.nkv;
            const int n = s_first[s + 1] - s_first[s];
            int count = 0;
            if (n > 0) {
                const int u_pair = s_first[s] * p.nkv + kvh * n;
                count = (u_pair + n - 1) / W - u_pair / W + 1;
            }
            p.piece_count[pair] = count;
        }
        const size_t rows_all = (size_t)p.n_tokens * p.nh;
        float* mml = mo + 4 * G * (HD / (G <= 4 ? 1 : (G <= 8 ? 2 : 4)));
        int consumed = 0, seq = seq0;
        bool ok = true;
        int u = u0;
        while (u < u_end && ok) {
            while (s_first[seq + 1] * p.nkv <= u) ++seq;
            const int n_seq = s_first[seq + 1] - s_first[seq];
            const int in_seq = u - s_first[seq] * p.nkv;
            const int kvh = in_seq / n_seq;
            const int t_rel = in_seq - kvh * n_seq;
            const int n_here = min(n_seq - t_rel, u_end - u);              // tiles of this piece
            const int u_pair = u - t_rel;
            const int piece = u / W - u_pair / W;                           // its place among the pair's pieces
            const int ctx = p.ctx_lens[seq];
            const int pos = ctx - 1;
            const int key_lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
            const int t_begin = key_lo / KV_TILE + t_rel, t_end = t_begin + n_here;
            const int tok = p.cu_seqlens[seq];
            bool valid[2];
            int head[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = quad + 8 * i;
                valid[i] = r < G;
                head[i] = kvh * G + (r < G ? r : 0);
            }
            uint32_t qa[HD / 16][4];
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const __nv_bfloat16* qp = p.q + ((size_t)tok * p.nh + head[i]) * HD + ks * 16 + tq * 2;
                    qa[ks][i] = valid[i] ? *reinterpret_cast<const uint32_t*>(qp) : 0u;
                    qa[ks][i + 2] = valid[i] ? *reinterpret_cast<const uint32_t*>(qp + 8) : 0u;
                }
            }
            float o[HD / 8][4];
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
            float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
            for (int t = t_begin; t < t_end; ++t, ++consumed) {
                const int stage = consumed % NST;
                if (!mbar_wait(full0 + 8 * stage, (consumed / NST) & 1, &abort_flag, 2)) { ok = false; break; }
                const unsigned char* ks = k_s + (size_t)stage * TMA_TILE_BYTES;
                const unsigned char* vs = v_s + (size_t)stage * TMA_TILE_BYTES;
                float s[2][4];
#pragma unroll
                for (int n = 0; n < 2; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    uint32_t b[4];
                    const int key_row = warp_n * 16 + (lane >> 4) * 8 + (lane & 7);
                    const int col = kk * 16 + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(b, ks + tma_swz(key_row, col));
                    mma_bf16(s[0], qa[kk], b[0], b[1]);
                    mma_bf16(s[1], qa[kk], b[2], b[3]);
                }
                const int key0 = t * KV_TILE + warp_n * 16 + tq * 2;
                float m_tile[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int n = 0; n < 2; ++n) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + n * 8 + (e & 1);
                        const bool see = key <= pos && key >= key_lo;
                        const float v = see ? s[n][e] * p.scale_log2e : -INFINITY;
                        s[n][e] = v;
                        m_tile[e >> 1] = fmaxf(m_tile[e >> 1], v);
                    }
                }
                float alpha[2], m_safe[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    m_tile[i] = fmaxf(m_tile[i], __shfl_xor_sync(0xffffffffu, m_tile[i], 1));
                    m_tile[i] = fmaxf(m_tile[i], __shfl_xor_sync(0xffffffffu, m_tile[i], 2));
                    const float m_new = fmaxf(m_run[i], m_tile[i]);
                    m_safe[i] = m_new == -INFINITY ? 0.f : m_new;
                    alpha[i] = exp2f(m_run[i] - m_safe[i]);
                    m_run[i] = m_new;
                }
                float l_tile[2] = {0.f, 0.f};
#pragma unroll
                for (int n = 0; n < 2; ++n) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float pv = exp2f(s[n][e] - m_safe[e >> 1]);
                        s[n][e] = pv;
                        l_tile[e >> 1] += pv;
                    }
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * alpha[i] + l_tile[i];
#pragma unroll
                for (int n = 0; n < HD / 8; ++n) {
                    o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
                    o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
                }
                uint32_t pa[4];
                pa[0] = pack_bf16(s[0][0], s[0][1]);
                pa[1] = pack_bf16(s[0][2], s[0][3]);
                pa[2] = pack_bf16(s[1][0], s[1][1]);
                pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
                for (int n2 = 0; n2 < HD / 16; ++n2) {
                    uint32_t b[4];
                    const int key_row = warp_n * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                    const int col = n2 * 16 + (lane >> 4) * 8;
                    ldmatrix_x4_trans(b, vs + tma_swz(key_row, col));
                    mma_bf16(o[2 * n2], pa, b[0], b[1]);
                    mma_bf16(o[2 * n2 + 1], pa, b[2], b[3]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * stage);      // this warp has read the stage for the last time
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
                l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
            }
            // ---- merge the four warps (their buffer lies behind the ring) and write the piece's partial result;
            // after a wait that gave up nothing is written, but every consumer still comes to both barriers
            // The buffer holds HD / passes columns of the group's rows at a time (one pass for up to four heads a
            // group, two up to eight, four beyond): so that three CTAs still fit an SM.
            const int passes = G <= 4 ? 1 : (G <= 8 ? 2 : 4), HDP = HD / passes;
            bool gave_up = false;
            for (int ps = 0; ps < passes; ++ps) {
                consumer_sync();                               // the merge before (of the piece before, of the pass before) has been read
                const bool good = abort_flag == 0 && ok;
                if (good) {
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int row = quad + 8 * i;
                        if (row >= G) continue;
#pragma unroll
                        for (int n = 0; n < HD / 8; ++n) {
                            if (n * 8 < ps * HDP || n * 8 >= (ps + 1) * HDP) continue;
                            float* dst = mo + ((size_t)warp_n * G + row) * HDP + (n * 8 - ps * HDP) + tq * 2;
                            dst[0] = o[n][2 * i]; dst[1] = o[n][2 * i + 1];
                        }
                        if (ps == 0 && tq == 0) {
                            mml[(warp_n * G + row) * 2] = m_run[i];
                            mml[(warp_n * G + row) * 2 + 1] = l_run[i];
                        }
                    }
                }
                consumer_sync();
                if (abort_flag != 0 || !ok) { gave_up = true; break; }
                for (int idx = tid; idx < G * HDP; idx += 128) {
                    const int row = idx / HDP, dd = idx - row * HDP, d = ps * HDP + dd;
                    float m_all = -INFINITY;
#pragma unroll
                    for (int w = 0; w < 4; ++w) m_all = fmaxf(m_all, mml[(w * G + row) * 2]);
                    const float m_s = m_all == -INFINITY ? 0.f : m_all;
                    float l_all = 0.f, acc = 0.f;
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const float f = exp2f(mml[(w * G + row) * 2] - m_s);
                        l_all += mml[(w * G + row) * 2 + 1] * f;
                        acc += mo[((size_t)w * G + row) * HDP + dd] * f;
                    }
                    const size_t prow = (size_t)piece * rows_all + (size_t)tok * p.nh + kvh * G + row;
                    p.part_o[prow * HD + d] = acc;
                    if (d == 0) { p.part_ml[prow * 2] = m_all; p.part_ml[prow * 2 + 1] = l_all; }
                }
            }
            if (gave_up) { ok = false; break; }
            u += n_here;
        }
    }
    __syncthreads();
    if (tid == 0 && abort_flag != 0 && status) atomicCAS(status, 0, abort_flag);
}
#endif   // RV_HAVE_TMA_DECODE

// Merge of the balanced kernel's pieces: one block per (sequence, query head).
__global__ void flash_balanced_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              const int* __restrict__ piece_count, const int* __restrict__ cu_seqlens,
                                              __nv_bfloat16* __restrict__ out, int n_tokens, int nh, int nkv, int num_seqs) {
    rv_pdl_launch_dependents();
    const int r = threadIdx.x / COMBINE_TPR, d = (threadIdx.x - r * COMBINE_TPR) * 4;
    const int item = blockIdx.x * COMBINE_ROWS + r;          // (sequence, query head)
    const bool live = r < COMBINE_ROWS && item < num_seqs * nh;
    const int seq = live ? item / nh : 0, head = live ? item - seq * nh : 0;
    const int tok = cu_seqlens[seq];
    const bool decode = cu_seqlens[seq + 1] - tok == 1;       // metadata of the step: read before the wait
    rv_pdl_wait();
    if (!live || !decode) return;
    const int pieces = piece_count[seq * nkv + head / (nh / nkv)];
    const size_t row = (size_t)tok * nh + head;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (pieces > 0) v = merge_splits4(part_o, part_ml, row, (size_t)n_tokens * nh, pieces, d);
    uint2 o2;
    o2.x = pack_bf16(v.x, v.y);
    o2.y = pack_bf16(v.z, v.w);
    *reinterpret_cast<uint2*>(out + row * HEAD_DIM + d) = o2;
}

// The most pieces a (sequence, kv head) pair can be cut into by `ctas` CTAs when no sequence has more
// than max_ctx keys: the caller sizes scratch as this * n_tokens * nh * (HEAD_DIM + 2) floats and
// piece_count as num_seqs * nkv ints.
RV_EXPORT int rv_flash_balanced_max_pieces(int max_ctx, int nkv, int ctas) {
    const int tiles = (max_ctx + KV_TILE - 1) / KV_TILE;
    const int bound = ctas / (nkv > 0 ? nkv : 1) + 2;       // W >= nkv * tiles of the longest sequence / ctas
    return tiles < bound ? (tiles < 1 ? 1 : tiles) : bound;
}

// Decode attention (sequences that bring one token; the others are left alone) with the work cut
// evenly over `ctas` CTAs (0: three per SM).  scratch, piece_count: see rv_flash_balanced_max_pieces.
RV_EXPORT int rv_flash_decode_balanced(const void* q, const void* cache, const int* block_tables, const int* cu_seqlens,
                                       const int* ctx_lens, void* out, float* scratch, int* piece_count, int max_pieces,
                                       int n_tokens, int num_seqs, int nh, int nkv, int hd, int page_size, int max_blocks,
                                       float scale, int window, int ctas, cudaStream_t stream) {
    if (hd != HEAD_DIM) return RV_ERR_UNSUPPORTED;
    if (n_tokens < 0 || num_seqs < 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || max_blocks <= 0 || max_pieces < 1)
        return RV_ERR_BAD_SIZE;
    if (page_size & (page_size - 1)) return RV_ERR_UNSUPPORTED;
    if (nh / nkv > 16 || num_seqs > BAL_MAX_SEQS) return RV_ERR_UNSUPPORTED;
    if (n_tokens == 0 || num_seqs == 0) return RV_OK;
    if (!scratch || !piece_count) return RV_ERR_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(out)) % 16)
        return RV_ERR_ALIGNMENT;
    BalancedParams p;
    p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.ctx_lens = ctx_lens;
    p.out = (__nv_bfloat16*)out;
    p.part_o = scratch;
    p.part_ml = scratch + (size_t)max_pieces * n_tokens * nh * HEAD_DIM;
    p.piece_count = piece_count;
    p.n_tokens = n_tokens; p.num_seqs = num_seqs; p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.max_blocks = max_blocks;
    p.max_pieces = max_pieces;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.window = window;
    if (ctas <= 0) ctas = 3 * rv_sm_count();
    const int merge_bytes = 4 * 16 * (HEAD_DIM + 2) * 4;
    const int smem = max(DECODE_STAGES * 2 * TILE_BYTES, merge_bytes);
    static RvPerDevice configured;
    if (int e = rv_configure_smem(configured, flash_decode_balanced_kernel<DECODE_STAGES>, smem)) return e;
    RV_LAUNCH_ST = rv_launch(flash_decode_balanced_kernel<DECODE_STAGES>, dim3(ctas), dim3(128), smem, stream, p);
    int st = rv_launch_status();
    if (st != RV_OK) return st;
    RV_LAUNCH_ST = rv_launch(flash_balanced_combine_kernel, dim3((num_seqs * nh + COMBINE_ROWS - 1) / COMBINE_ROWS), dim3(128), 0, stream,
                             (const float*)p.part_o, (const float*)p.part_ml, (const int*)piece_count, cu_seqlens, p.out,
                             n_tokens, nh, nkv, num_seqs);
    return rv_launch_status();
}

template <int WARPS_M, int WARPS_N, int NSTAGES>
static int launch_flash(const FlashParams& p, int num_seqs, cudaStream_t stream) {
    const int merge_bytes = WARPS_N > 1 ? WARPS_N * 16 * (HEAD_DIM + 2) * 4 : 0;
    const int smem = max(NSTAGES * 2 * TILE_BYTES, merge_bytes);
    static RvPerDevice configured;
    if (int e = rv_configure_smem(configured, flash_paged_kernel<WARPS_M, WARPS_N, NSTAGES>, smem)) return e;
    const dim3 grid(p.row_tiles * p.num_splits, p.nkv, num_seqs);
    RV_LAUNCH_ST = rv_launch(flash_paged_kernel<WARPS_M, WARPS_N, NSTAGES>, dim3(grid), dim3(WARPS_M * WARPS_N * 32), smem, stream, p);
    return rv_launch_status();
}

RV_EXPORT int rv_flash_head_dim() { return HEAD_DIM; }

// How many floats of scratch `rv_flash_attention` needs for `num_splits` > 1.
RV_EXPORT long long rv_flash_scratch_floats(int n_tokens, int nh, int num_splits) {
    return num_splits > 1 ? (long long)num_splits * n_tokens * nh * (HEAD_DIM + 2) : 0;
}

// mode 0: prefill / mixed tiling (64 rows per CTA); mode 1: decode tiling (16 rows, warps split
// the keys), for steps in which the selected sequences bring one token each.
// scratch: float buffer of rv_flash_scratch_floats(...) elements when num_splits > 1.
RV_EXPORT int rv_flash_attention(const void* q, const void* cache, const int* block_tables, const int* cu_seqlens,
                                 const int* ctx_lens, void* out, float* scratch, int n_tokens, int num_seqs,
                                 int nh, int nkv, int hd, int page_size, int max_blocks, float scale, int window,
                                 int mode, int max_q_len, int num_splits, int q_filter, cudaStream_t stream) {
    if (hd != HEAD_DIM) return RV_ERR_UNSUPPORTED;
    if (n_tokens < 0 || num_seqs < 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || max_blocks <= 0 ||
        max_q_len <= 0 || num_splits < 1)
        return RV_ERR_BAD_SIZE;
    if (page_size & (page_size - 1)) return RV_ERR_UNSUPPORTED;
    if (num_seqs > 65535 || nkv > 65535) return RV_ERR_BAD_SIZE;
    if (n_tokens == 0 || num_seqs == 0) return RV_OK;
    if (num_splits > 1 && scratch == nullptr) return RV_ERR_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(out)) % 16)
        return RV_ERR_ALIGNMENT;
    FlashParams p;
    p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.ctx_lens = ctx_lens;
    p.out = (__nv_bfloat16*)out;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + (size_t)num_splits * n_tokens * nh * HEAD_DIM : nullptr;
    p.n_tokens = n_tokens; p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.max_blocks = max_blocks;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.window = window; p.num_splits = num_splits; p.q_filter = q_filter;
    const int G = nh / nkv;
    const int m_tile = mode == 1 ? 16 : 64;
    p.row_tiles = (max_q_len * G + m_tile - 1) / m_tile;
    int st = mode == 1 ? launch_flash<1, 4, DECODE_STAGES>(p, num_seqs, stream) : launch_flash<4, 1, 2>(p, num_seqs, stream);
    if (st != RV_OK) return st;
    if (num_splits > 1) {
        RV_LAUNCH_ST = rv_launch(flash_combine_kernel, dim3((n_tokens * nh + COMBINE_ROWS - 1) / COMBINE_ROWS), dim3(128), 0, stream,
                                 p.part_o, p.part_ml, p.out, n_tokens * nh, num_splits);
        return rv_launch_status();
    }
    return RV_OK;
}

// The TMA-fed decode kernel for the sequences of a step that bring one token (q_filter 1) or for
// a step of such sequences only (q_filter 0 with max_q_len 1).  Same arguments as rv_flash_attention
// plus the number of pages of the cache layer (for the tensor map), the status word of bounded
// waits and `early` (request keys before griddepcontrol.wait).  Refuses (RV_ERR_UNSUPPORTED) head
// sizes other than 64 and 128 and pages of fewer than 8 keys: the caller falls back to rv_flash_attention.
RV_EXPORT int rv_flash_decode_tma(const void* q, const void* cache, long long num_pages, const int* block_tables,
                                  const int* cu_seqlens, const int* ctx_lens, void* out, float* scratch, int n_tokens,
                                  int num_seqs, int nh, int nkv, int hd, int page_size, int max_blocks, float scale,
                                  int window, int max_q_len, int num_splits, int q_filter, int* status, int early,
                                  cudaStream_t stream) {
#ifdef RV_HAVE_TMA_DECODE
    if (hd != HEAD_DIM) return RV_ERR_UNSUPPORTED;
    if (n_tokens < 0 || num_seqs < 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || max_blocks <= 0 ||
        max_q_len <= 0 || num_splits < 1 || num_pages <= 0)
        return RV_ERR_BAD_SIZE;
    if ((page_size & (page_size - 1)) || page_size < 8) return RV_ERR_UNSUPPORTED;
    if (num_seqs > 65535 || nkv > 65535) return RV_ERR_BAD_SIZE;
    if (n_tokens == 0 || num_seqs == 0) return RV_OK;
    if (num_splits > 1 && scratch == nullptr) return RV_ERR_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(out)) % 16)
        return RV_ERR_ALIGNMENT;
    alignas(64) CUtensorMap map_kv;
    int st = rv_make_bf16_map(&map_kv, cache, num_pages * 2 * nkv * page_size, HEAD_DIM, page_size < KV_TILE ? page_size : KV_TILE);
    if (st != RV_OK) return st;
    FlashParams p;
    p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.ctx_lens = ctx_lens;
    p.out = (__nv_bfloat16*)out;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + (size_t)num_splits * n_tokens * nh * HEAD_DIM : nullptr;
    p.n_tokens = n_tokens; p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.max_blocks = max_blocks;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.window = window; p.num_splits = num_splits; p.q_filter = q_filter;
    const int G = nh / nkv;
    p.row_tiles = (max_q_len * G + 15) / 16;
    const int smem = 2 * TMA_STAGES * TMA_TILE_BYTES + 1024;
    static RvPerDevice configured;
    if (int e = rv_configure_smem(configured, flash_decode_tma_kernel<TMA_STAGES>, smem)) return e;
    const dim3 grid(p.row_tiles * p.num_splits, p.nkv, num_seqs);
    RV_LAUNCH_ST = rv_launch(flash_decode_tma_kernel<TMA_STAGES>, grid, dim3(TMA_THREADS), smem, stream, map_kv, p, status, early);
    st = rv_launch_status();
    if (st != RV_OK) return st;
    if (num_splits > 1) {
        RV_LAUNCH_ST = rv_launch(flash_combine_kernel, dim3((n_tokens * nh + COMBINE_ROWS - 1) / COMBINE_ROWS), dim3(128), 0, stream,
                                 p.part_o, p.part_ml, p.out, n_tokens * nh, num_splits);
        return rv_launch_status();
    }
    return RV_OK;
#else
    return RV_ERR_UNSUPPORTED;
#endif
}

// The evenly cut decode kernel fed by TMA (head sizes 64 and 128, pages of at least 8 keys; else
// RV_ERR_UNSUPPORTED and the caller takes rv_flash_decode_balanced).  Same arguments, plus the number of pages
// of the cache layer (for the tensor map) and the status word of the bounded waits.  ctas <= 0: as many as
// stay resident, which rv_flash_balanced_tma_ctas tells the caller, who sizes scratch by it.
#ifdef RV_HAVE_TMA_DECODE
static int balanced_tma_smem(int G) {       // the ring, the merge buffer (HEAD_DIM / passes columns of G rows of four warps) and its maxima and sums
    const int passes = G <= 4 ? 1 : (G <= 8 ? 2 : 4);
    return 2 * TMA_STAGES * TMA_TILE_BYTES + 4 * G * (HEAD_DIM / passes + 2) * 4 + 1024;
}
#endif
RV_EXPORT int rv_flash_balanced_tma_ctas(int nh, int nkv) {
#ifdef RV_HAVE_TMA_DECODE
    if (nh <= 0 || nkv <= 0 || nh % nkv || nh / nkv > 16) return 0;
    const int smem = balanced_tma_smem(nh / nkv);
    static RvPerDevice configured;
    if (rv_configure_smem(configured, flash_decode_balanced_tma_kernel<TMA_STAGES>, balanced_tma_smem(16))) return 0;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, flash_decode_balanced_tma_kernel<TMA_STAGES>, TMA_THREADS, smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return per_sm * rv_sm_count();
#else
    return 0;
#endif
}
RV_EXPORT int rv_flash_decode_balanced_tma(const void* q, const void* cache, long long num_pages, const int* block_tables,
                                           const int* cu_seqlens, const int* ctx_lens, void* out, float* scratch,
                                           int* piece_count, int max_pieces, int n_tokens, int num_seqs, int nh, int nkv,
                                           int hd, int page_size, int max_blocks, float scale, int window, int ctas,
                                           int* status, cudaStream_t stream) {
#ifdef RV_HAVE_TMA_DECODE
    if (hd != HEAD_DIM) return RV_ERR_UNSUPPORTED;
    if (n_tokens < 0 || num_seqs < 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || max_blocks <= 0 || max_pieces < 1 ||
        num_pages <= 0)
        return RV_ERR_BAD_SIZE;
    if ((page_size & (page_size - 1)) || page_size < 8) return RV_ERR_UNSUPPORTED;
    if (nh / nkv > 16 || num_seqs > BAL_TMA_MAX_SEQS) return RV_ERR_UNSUPPORTED;
    if (n_tokens == 0 || num_seqs == 0) return RV_OK;
    if (!scratch || !piece_count) return RV_ERR_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(out)) % 16)
        return RV_ERR_ALIGNMENT;
    alignas(64) CUtensorMap map_kv;
    int st = rv_make_bf16_map(&map_kv, cache, num_pages * 2 * nkv * page_size, HEAD_DIM, page_size < KV_TILE ? page_size : KV_TILE);
    if (st != RV_OK) return st;
    if (ctas <= 0) ctas = rv_flash_balanced_tma_ctas(nh, nkv);
    if (ctas <= 0) return RV_ERR_UNSUPPORTED;
    BalancedParams p;
    p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.ctx_lens = ctx_lens;
    p.out = (__nv_bfloat16*)out;
    p.part_o = scratch;
    p.part_ml = scratch + (size_t)max_pieces * n_tokens * nh * HEAD_DIM;
    p.piece_count = piece_count;
    p.n_tokens = n_tokens; p.num_seqs = num_seqs; p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.max_blocks = max_blocks;
    p.max_pieces = max_pieces;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.window = window;
    const int smem = balanced_tma_smem(nh / nkv);
    static RvPerDevice configured;
    if (int e = rv_configure_smem(configured, flash_decode_balanced_tma_kernel<TMA_STAGES>, balanced_tma_smem(16))) return e;
    RV_LAUNCH_ST = rv_launch(flash_decode_balanced_tma_kernel<TMA_STAGES>, dim3(ctas), dim3(TMA_THREADS), smem, stream, map_kv, p, status);
    st = rv_launch_status();
    if (st != RV_OK) return st;
    RV_LAUNCH_ST = rv_launch(flash_balanced_combine_kernel, dim3((num_seqs * nh + COMBINE_ROWS - 1) / COMBINE_ROWS), dim3(128), 0, stream,
                             (const float*)p.part_o, (const float*)p.part_ml, (const int*)piece_count, cu_seqlens, p.out,
                             n_tokens, nh, nkv, num_seqs);
    return rv_launch_status();
#else
    return RV_ERR_UNSUPPORTED;
#endif
}

// ---------------------------------------------------------------------------------------------
// rv_flash_attention_static: the same attention, for callers that may not allocate.
// Declared and documented in attention_flash_static.h.  It has no counterpart in the reference.
//
// The split-key partials live in a file-scope device array instead of a caller's buffer.  In host
// code the array's name is only a stand-in for the symbol, not an address a kernel can use, so
// its device address is fetched once per device with cudaGetSymbolAddress (with that device
// current) and kept; kernels get that address.
#include "attention_flash_static.h"
#include <stdarg.h>
#include <stdio.h>

static __device__ __align__(256) float g_static_scratch[RV_FLASH_STATIC_SCRATCH_FLOATS];

#define RV_STATIC_MAX_DEVICES 64
static float* g_static_scratch_addr[RV_STATIC_MAX_DEVICES];   // zero-initialised: not set up yet

static void static_fail(char* err, int err_len, const char* fmt, ...) {
    if (!err || err_len <= 0) return;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, (size_t)err_len, fmt, ap);
    va_end(ap);
}

RV_EXPORT int rv_flash_attention_static(const void* q, const void* cache, const int* block_tables,
                                        const int* cu_seqlens, const int* ctx_lens, void* out, int n_tokens,
                                        int num_seqs, int nh, int nkv, int hd, int page_size, int max_blocks,
                                        float scale, int window, int mode, int max_q_len, int num_splits,
                                        cudaStream_t stream, char* err, int err_len) {
    if (err && err_len > 0) err[0] = 0;
    if (num_splits < 1 || n_tokens < 0 || nh <= 0) {
        static_fail(err, err_len, "rv_flash_attention_static: bad sizes (num_splits %d, n_tokens %d, num_heads %d)", num_splits, n_tokens, nh);
        return RV_ERR_BAD_SIZE;
    }
    const long long need = rv_flash_scratch_floats(n_tokens, nh, num_splits);
    if (need > (long long)RV_FLASH_STATIC_SCRATCH_FLOATS) {
        static_fail(err, err_len, "rv_flash_attention_static: this call needs %lld floats of scratch, the built-in "
                    "array holds %lld; use fewer key splits or rv_flash_attention with a buffer of your own",
                    need, (long long)RV_FLASH_STATIC_SCRATCH_FLOATS);
        return RV_ERR_SCRATCH_TOO_LARGE;
    }
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= RV_STATIC_MAX_DEVICES) {
        static_fail(err, err_len, "rv_flash_attention_static: cannot use device %d (CUDA error %d)", device, (int)e);
        return e != cudaSuccess ? (int)e : RV_ERR_UNSUPPORTED;
    }
    if (g_static_scratch_addr[device] == nullptr) {
        // first call on this device: look the array's device address up (this may load the
        // module, which is why the first call belongs before any stream capture)
        float* addr = nullptr;
        e = cudaGetSymbolAddress((void**)&addr, g_static_scratch);
        if (e != cudaSuccess || addr == nullptr) {
            static_fail(err, err_len, "rv_flash_attention_static: cudaGetSymbolAddress failed on device %d (CUDA error %d)",
                        device, (int)e);
            return e != cudaSuccess ? (int)e : RV_ERR_UNSUPPORTED;
        }
        g_static_scratch_addr[device] = addr;
    }
    // Nothing in the scratch has to be zero at entry: for every row that the sequences cover, every
    // element the merge kernel reads was written by the attention kernel of the same call (empty key
    // ranges write m = -inf, l = 0).  Rows outside the sequences are undefined (see the header).
    const int st = rv_flash_attention(q, cache, block_tables, cu_seqlens, ctx_lens, out,
                                      num_splits > 1 ? g_static_scratch_addr[device] : nullptr, n_tokens, num_seqs,
                                      nh, nkv, hd, page_size, max_blocks, scale, window, mode, max_q_len, num_splits,
                                      /*q_filter=*/0, stream);
    if (st != RV_OK) static_fail(err, err_len, "rv_flash_attention_static: the attention launch was refused or failed (code %d)", st);
    return st;
}
