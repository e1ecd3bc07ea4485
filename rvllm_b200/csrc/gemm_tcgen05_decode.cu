// bfloat16 linear layer for few rows (decode) on the fifth-generation tensor cores:
//     out[M, N] = x[M, K] . W[N, K]^T (+ bias[N]) (+ residual[M, N]),       M <= 128,
// or GATED with W rows [gate (N/2) | up (N/2)]:  out[M, N/2] = silu(x Wg^T) * (x Wu^T).
//
// The product is computed transposed: the WEIGHTS are the 128-row A operand of tcgen05.mma and
// the batch is its N dimension (16 to 128 columns of tensor memory), so a CTA streams a tile of
// 128 output features through a TMA pipeline and every weight byte is read from HBM exactly once
// whatever the batch size.  Small N would leave most SMs idle, so K is also split over CTAs;
// the CTAs of a tile write float partials to scratch memory, and the CTA that arrives last (an
// atomic counter per tile, no spinning) adds them in split order and runs the epilogue.  The sum
// of a row therefore does not depend on which CTA came last, nor on the other rows of the batch.
//
//   warp 0   TMA producer (one thread): weight tile 128 x 64 and activation tile MB x 64 per
//            stage, 128-byte swizzle, 4 stages;
//   warp 1   MMA issuer (one thread): tcgen05.mma M = 128, N = MB, K = 16; tcgen05.commit frees
//            stages and finally publishes the accumulator;
//   warps 2-5  epilogue: tcgen05.ld of each thread's feature row, split reduction, bias,
//            residual, SiLU-gate, rounding, coalesced stores.
// A third epilogue serves the q/k/v product of an attention layer: W rows are [q heads | k heads |
// v heads]; the tile's sums are rounded to bfloat16 as a separate product would store them, then
// the bias is added, q and k are rotated by the token's position (pairs i, i + head_dim/2, which
// lie in one tile because 128 is a multiple of head_dim), q goes to its output and k and v go
// straight into the token's slot of the paged cache - one kernel and one pass less per layer.
// With `norm_gamma` set the activations arrive unnormalised and the kernel applies RMSNorm itself
// (at most 16 rows): the epilogue warps, idle during the main loop, first form each row's
// 1 / sqrt(mean(x^2) + eps) from global memory, then scale every activation tile in shared memory
// by it and by gamma as soon as its TMA load has landed, and hand the tile to the MMA warp through a
// second barrier per stage.  The norm kernel and its place in the chain of launches are saved.
// For up to 64 rows and up to 8 splits the CTAs of a tile are launched as a thread-block cluster.  The
// rows are dealt out to the CTAs, ceil(M / splits) each; every CTA writes its partial of a row into
// the shared memory of the CTA that owns the row (st.shared::cluster), and one cluster barrier later
// each CTA adds its rows' partials in split order and runs their epilogue - no round trip through L2,
// no fence, no atomic.  Every thread of every CTA reaches the cluster barrier on every path.
// Every mbarrier wait is bounded (see gemm_tcgen05.cu); no multicast.
//
// Shapes: the five products of a layer and the LM head at decode time
// (v3/crates/rvllm-runtime/src/layer_exec.rs:240-266,433-444,478-488,511-522 and
// bring_up.rs:648-658 of the reference, which calls cuBLASLt there).
#include "common.cuh"
#include "tcgen05.cuh"

#define TILE_F 128           // output features per tile (UMMA M)
#define BK 64
// stages of the TMA ring: four, or three for 33 to 64 rows, whose wider activation tiles and cluster buffers
// would otherwise leave room for only one CTA per SM
#define STAGES_FOR(MB) ((MB) > 32 && (MB) <= 64 ? 3 : 4)
#define UMMA_K 16
#define A_BYTES (TILE_F * BK * 2)
#define NUM_THREADS 192
#define MAX_NORM_K 8192      // longest K range of one CTA for which the fused norm keeps gamma in shared memory

struct DecodeGemmParams {
    void* out;
    const __nv_bfloat16* residual;
    const void* bias;
    int bias_dtype;
    float* scratch;          // [tiles, splits, MB, 128] float partials (splits > 1)
    int* counters;           // [tiles], zero between launches
    int* status;
    int M, N, K;
    int out_f32, gated;
    int splits, n_tiles;
    int cluster;             // 1: the CTAs of a tile are a thread-block cluster and add their partials in the
                             // cluster's shared memory (M <= 64, 2 <= splits <= 8); scratch and counters unused
    int cluster_rows;        // rows that each CTA of the cluster finishes: ceil(M / splits)
    int k_rotate;            // != 0: tile t starts its K loop at k block (t * k_rotate) mod its count, so that the CTAs of a
                             // wave ask for different blocks of the activations at a time, not all for the same lines of L2
    int l2_ahead;            // k blocks beyond the shared-memory stages whose weights are asked into L2 before the wait
    // rotary epilogue (q_out != nullptr): N = (nh + 2 nkv) * hd, 128 % hd == 0
    __nv_bfloat16* q_out;            // [M, nh * hd]
    __nv_bfloat16* kv_cache;         // [pages, 2, nkv, page_size, hd]
    const int* positions;            // [M]
    const int* slot_mapping;         // [M], < 0: the row writes no key or value
    const float* cos_t;              // [table_rows, hd / 2] or nullptr (no rotation)
    const float* sin_t;
    int nh, nkv, hd, page_size, table_rows;
    // fused RMSNorm of the activations (norm_gamma != nullptr): x_raw are the rows the map_x loads
    const void* norm_gamma;          // [K]
    const __nv_bfloat16* x_raw;      // [M, K]
    int norm_gamma_dtype;
    float norm_eps;
};

__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of `addr` (a shared-memory address of this CTA) in CTA `rank`.
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// One bulk copy from this CTA's shared memory into another CTA's of the cluster; its bytes are counted on a barrier
// of the receiving CTA (both given as addresses in the cluster's shared window).
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t dst, uint32_t src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "r"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// The partials of a tile added up and the epilogue run in one pass, by the epilogue warps of the CTA
// that finishes the tile: four neighbouring features per thread (16-byte reads of the partials,
// 8-byte reads of the residual, 8- or 16-byte stores), four rows and four splits in flight at a
// time.  A row is summed in split order, whatever the batch holds.  The partial of (split s, row m)
// starts at parts + (s * part_rows + m - row_begin) * 128, in scratch memory or in the CTA's shared
// memory; the rows [row_begin, row_end) are finished.
// (volatile asm on purpose: plain loads let the compiler hoist all of a thread's loads and spend 47 more registers)
template <bool IN_SMEM>
__device__ __forceinline__ float4 load_part(const float* src) {
    float4 v;
    if (IN_SMEM)
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_u32(src)) : "memory");
    else
        asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(src) : "memory");
    return v;
}

// SiLU(g) * u.  For a bfloat16 result the hardware's approximations of 2^x and 1/x (two units in the last
// place of a float, a 4000th of the result's own rounding step) save half of the epilogue's instructions.
__device__ __forceinline__ float silu_gate(float g, float u, bool exact) {
    return exact ? g / (1.0f + expf(-g)) * u : __fdividef(g, 1.0f + __expf(-g)) * u;
}

template <int MB, bool IN_SMEM>
__device__ __forceinline__ void finish_from_parts(const DecodeGemmParams& p, int tile, int et, const float* parts,
                                                  int part_rows, int row_begin, int row_end, int* row_pos, int* row_slot) {
    const int fq = et & 31, rg = et >> 5;
    const int n0 = tile * TILE_F + 4 * fq;
    const float* base = parts + 4 * fq;
    const bool vec = (p.N & 3) == 0 && n0 + 3 < p.N;
    if (p.q_out) {
        if (et < p.M) {
            const int pos = p.positions[et];
            row_pos[et] = pos < 0 ? 0 : (pos >= p.table_rows ? p.table_rows - 1 : pos);
            row_slot[et] = p.slot_mapping[et];
        }
        epi_sync();
    }
    float bias4[4] = {0.f, 0.f, 0.f, 0.f};
    if (p.bias) {
#pragma unroll
        for (int e = 0; e < 4; ++e) if (n0 + e < p.N) bias4[e] = rv_load_param(p.bias, p.bias_dtype, n0 + e);
    }
    for (int m0 = row_begin + rg; m0 < row_end; m0 += 16) {
        float4 acc[4];
        uint2 res[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            res[j] = make_uint2(0u, 0u);
            const int m = m0 + 4 * j;
            if (p.residual && vec && m < row_end)
                res[j] = __ldg(reinterpret_cast<const uint2*>(p.residual + (size_t)m * p.N + n0));
        }
        for (int s0 = 0; s0 < p.splits; s0 += 4) {
            float4 t[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    t[j][i] = (m0 + 4 * j < row_end && s0 + i < p.splits)
                                  ? load_part<IN_SMEM>(base + ((size_t)(s0 + i) * part_rows + m0 + 4 * j - row_begin) * TILE_F)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[j].x += t[j][i].x; acc[j].y += t[j][i].y; acc[j].z += t[j][i].z; acc[j].w += t[j][i].w;
                }
        }
        if (p.q_out) {
            // rotary epilogue: hd is a power of two >= 8 and N a multiple of it, so the four
            // features lie in one half of one head and their partners (hd / 2 further or
            // nearer) are held by the lane hd / 8 away; every lane takes part in the exchange
            const int hd = p.hd, half = hd >> 1;
            const int head = n0 / hd, d = n0 - head * hd;
            const bool live = n0 < p.N;
            const bool is_q = head < p.nh, is_k = !is_q && head < p.nh + p.nkv;
            const bool first = d < half;
            const int i0 = first ? d : d - half;
            const int kvh = is_k ? head - p.nh : head - p.nh - p.nkv;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int m = m0 + 4 * j;
                const bool row_ok = m < row_end;                 // uniform in the warp
                float own[4] = {acc[j].x, acc[j].y, acc[j].z, acc[j].w}, other[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    own[e] = own[e] + bias4[e];                       // float sums throughout: one rounding, at the store
                    other[e] = __shfl_xor_sync(0xffffffffu, own[e], hd >> 3);
                }
                if (!row_ok || !live) continue;
                float v[4] = {own[0], own[1], own[2], own[3]};
                if ((is_q || is_k) && p.cos_t) {
                    const float4 c = __ldg(reinterpret_cast<const float4*>(p.cos_t + (size_t)row_pos[m] * half + i0));
                    const float4 sn = __ldg(reinterpret_cast<const float4*>(p.sin_t + (size_t)row_pos[m] * half + i0));
                    const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        v[e] = first ? own[e] * cc[e] - other[e] * ss[e] : other[e] * ss[e] + own[e] * cc[e];
                }
                uint2 o2;
                o2.x = pack_bf16x2(v[0], v[1]);
                o2.y = pack_bf16x2(v[2], v[3]);
                if (is_q) {
                    *reinterpret_cast<uint2*>(p.q_out + (size_t)m * p.nh * hd + n0) = o2;
                } else {
                    const int slot = row_slot[m];
                    if (slot >= 0) {
                        const int page = slot / p.page_size, off = slot - page * p.page_size;
                        *reinterpret_cast<uint2*>(p.kv_cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * p.nkv + kvh) * p.page_size + off) * hd + d) = o2;
                    }
                }
            }
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + 4 * j;
            if (m >= row_end || n0 >= p.N) continue;
            float v[4] = {acc[j].x + bias4[0], acc[j].y + bias4[1], acc[j].z + bias4[2], acc[j].w + bias4[3]};
            if (vec) {
                if (p.residual) {
                    const __nv_bfloat16* re = reinterpret_cast<const __nv_bfloat16*>(&res[j]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[e] += __bfloat162float(re[e]);
                }
                if (p.out_f32) {
                    *reinterpret_cast<float4*>((float*)p.out + (size_t)m * p.N + n0) = make_float4(v[0], v[1], v[2], v[3]);
                } else {
                    uint2 o2;
                    o2.x = pack_bf16x2(v[0], v[1]);
                    o2.y = pack_bf16x2(v[2], v[3]);
                    *reinterpret_cast<uint2*>((__nv_bfloat16*)p.out + (size_t)m * p.N + n0) = o2;
                }
            } else {
                for (int e = 0; e < 4 && n0 + e < p.N; ++e) {
                    float w = v[e];
                    if (p.residual) w += __bfloat162float(p.residual[(size_t)m * p.N + n0 + e]);
                    if (p.out_f32) ((float*)p.out)[(size_t)m * p.N + n0 + e] = w;
                    else ((__nv_bfloat16*)p.out)[(size_t)m * p.N + n0 + e] = __float2bfloat16_rn(w);
                }
            }
        }
    }
}

template <int MB>
__global__ void __launch_bounds__(NUM_THREADS, (MB <= 16 || MB == 64) ? 3 : 2)
gemm_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const DecodeGemmParams p_in) {
    // More than 128 rows (MB = 128 only): blockIdx.y is a block of 128 rows, which this CTA treats as a
    // product of its own - the rows' pointers moved on, M cut to the block.  The other widths see the
    // parameters as they came.
    DecodeGemmParams p_blk;
    int x_row0 = 0;
    if constexpr (MB == 128) {
        p_blk = p_in;
        x_row0 = (int)blockIdx.y * MB;
        if (x_row0 > 0) {
            const size_t r0 = (size_t)x_row0;
            const size_t n_out = p_in.gated ? (size_t)(p_in.N >> 1) : (size_t)p_in.N;
            p_blk.out = p_in.out_f32 ? (void*)((float*)p_in.out + r0 * n_out) : (void*)((__nv_bfloat16*)p_in.out + r0 * n_out);
            if (p_in.residual) p_blk.residual = p_in.residual + r0 * p_in.N;
            if (p_in.q_out) {
                p_blk.q_out = p_in.q_out + r0 * p_in.nh * p_in.hd;
                p_blk.positions = p_in.positions + r0;
                p_blk.slot_mapping = p_in.slot_mapping + r0;
            }
        }
        p_blk.M = min(MB, p_in.M - x_row0);
    }
    const DecodeGemmParams& p = (MB == 128) ? p_blk : p_in;
    constexpr int STAGES = STAGES_FOR(MB);
    constexpr int B_BYTES = MB * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int TMEM_COLS = MB < 32 ? 32 : MB;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[3 * STAGES + 2];     // full, empty, accumulator ready, normalised, partials arrived
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;
    __shared__ int is_last;
    __shared__ int row_pos[128], row_slot[128];
    __shared__ float norm_red[4][16], norm_rstd[16];

    rv_pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]), tfull = smem_u32(&bars[2 * STAGES]);
    const uint32_t normed0 = smem_u32(&bars[2 * STAGES + 1]);
    const uint32_t xbar = smem_u32(&bars[3 * STAGES + 1]);     // the other CTAs' partials of this CTA's rows have arrived
    const bool fused_norm = p.norm_gamma != nullptr;

    const int tile = blockIdx.x / p.splits, split = blockIdx.x - tile * p.splits;
    const int num_kb = (p.K + BK - 1) / BK;
    const int per = (num_kb + p.splits - 1) / p.splits;
    const int kb0 = split * per, kb1 = min(num_kb, kb0 + per);
    const int n_kb = kb1 > kb0 ? kb1 - kb0 : 0;
    const int rot = (p.k_rotate && n_kb > 1) ? (int)(((unsigned)tile * (unsigned)p.k_rotate) % (unsigned)n_kb) : 0;
    // the i-th k block of this CTA's loop: its range, begun at `rot` and wrapped around
    auto kb_at = [&](int i) { const int r = i + rot; return kb0 + (r >= n_kb ? r - n_kb : r); };
    const int half_n = p.N >> 1;
    // first weight row of the tile's (two) halves
    const int row_a = p.gated ? tile * (TILE_F / 2) : tile * TILE_F;
    const int row_b = p.gated ? half_n + tile * (TILE_F / 2) : tile * TILE_F + TILE_F / 2;
    const int early = min(STAGES, n_kb);

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&map_w);
        tma_prefetch_descriptor(&map_x);
        abort_flag = 0;
        is_last = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); mbar_init(normed0 + 8 * s, 4); }
        mbar_init(tfull, 1);
        mbar_init(xbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // The weights are written by no kernel of a step: the first stages' weight tiles are requested
        // at once, by the thread that has just set the barriers up - before the tensor memory is
        // allocated, before the CTA's first barrier and before the wait for the previous kernel, whose
        // tail this overlaps.  The activations follow after that wait; a stage's barrier completes when
        // both have landed.
        for (int i = 0; i < early; ++i) {
            const uint32_t a_dst = smem_u32(tiles + (size_t)i * STAGE_BYTES);
            const uint32_t bar = full0 + 8 * i;
            mbar_expect_tx(bar, STAGE_BYTES);
            tma_load_2d(a_dst, &map_w, kb_at(i) * BK, row_a, bar);
            tma_load_2d(a_dst + A_BYTES / 2, &map_w, kb_at(i) * BK, row_b, bar);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    // A CTA's shared memory and its barrier may be written from another CTA of the cluster only once it runs and
    // has set them up: every thread arrives here; the epilogue warps wait before partials are sent, the others at the end.
    if (p.cluster) cluster_arrive();

    // cluster reduction: [splits][cluster_rows][128 features] floats behind the stages (and gamma),
    // at the same offset in every CTA of the cluster
    float* red = reinterpret_cast<float*>(tiles + (size_t)STAGES * STAGE_BYTES + (fused_norm ? (size_t)per * BK * 4 : 0));

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0, issued = 0;
            uint32_t phase = 0;
            bool ok = true;
            // (the first stages' weights were requested during the set-up above) ... and the weights of
            // the k blocks after them are asked into L2: while this kernel waits
            // for its predecessor (a norm, the merge of the attention's key splits) the memory is idle
            for (int i = early; i < min(n_kb, early + p.l2_ahead); ++i) {
                tma_prefetch_2d(&map_w, kb_at(i) * BK, row_a);
                tma_prefetch_2d(&map_w, kb_at(i) * BK, row_b);
            }
            rv_pdl_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(smem_u32(tiles + (size_t)i * STAGE_BYTES) + A_BYTES, &map_x, kb_at(i) * BK, x_row0, full0 + 8 * i);
            issued = early;
            stage = early % STAGES;
            phase = early == STAGES ? 1 : 0;
            for (int i = early; i < n_kb; ++i) {
                const int kb = kb_at(i);
                if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, &abort_flag, 1)) { ok = false; break; }
                const uint32_t a_dst = smem_u32(tiles + (size_t)stage * STAGE_BYTES);
                const uint32_t bar = full0 + 8 * stage;
                mbar_expect_tx(bar, STAGE_BYTES);
                tma_load_2d(a_dst, &map_w, kb * BK, row_a, bar);
                tma_load_2d(a_dst + A_BYTES / 2, &map_w, kb * BK, row_b, bar);
                tma_load_2d(a_dst + A_BYTES, &map_x, kb * BK, x_row0, bar);
                ++issued;
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            if (!ok) {
                const int pending = issued < STAGES ? issued : STAGES;
                for (int i = 0; i < pending; ++i) {
                    int s = stage - 1 - i;
                    uint32_t ph = phase;
                    while (s < 0) { s += STAGES; ph ^= 1; }
                    for (uint32_t it = 0; it < (1u << 20); ++it)
                        if (mbar_try(full0 + 8 * s, ph)) break;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(TILE_F, MB);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int i = 0; i < n_kb; ++i) {
                if (!mbar_wait((fused_norm ? normed0 : full0) + 8 * stage, phase, &abort_flag, 3)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t a_addr = smem_u32(tiles + (size_t)stage * STAGE_BYTES);
                const uint64_t da = umma_desc(a_addr), db = umma_desc(a_addr + A_BYTES);
#pragma unroll
                for (int j = 0; j < BK / UMMA_K; ++j)
                    tcgen05_mma_bf16(tmem_base, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc, i > 0 || j != 0);
                tcgen05_commit(empty0 + 8 * stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok) tcgen05_commit(tfull);
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;
        const int f = quarter * 32 + lane;                  // feature row of this thread within the tile
        const int et = (warp - 2) * 32 + lane;              // 0..127 among the epilogue threads
        const bool have = kb1 > kb0;
        float* gam = reinterpret_cast<float*>(tiles + (size_t)STAGES * STAGE_BYTES);   // gamma of this CTA's K range
        if (fused_norm) {
            // gamma is a weight: it is fetched before the wait for the previous kernel
            const int nk = (kb1 - kb0) * BK;
            for (int i = et; i < nk; i += 128) {
                const int k = kb0 * BK + i;
                gam[i] = k < p.K ? rv_load_param(p.norm_gamma, p.norm_gamma_dtype, k) : 0.f;
            }
        }
        rv_pdl_wait();
        if (fused_norm) {
            // ---- each row's 1 / sqrt(mean(x^2) + eps), four rows' loads in flight together
            const int cpr = p.K >> 3;                       // 16-byte pieces per row
            for (int m0 = 0; m0 < p.M; m0 += 4) {
                float ss[4] = {0.f, 0.f, 0.f, 0.f};
                for (int c = et; c < cpr; c += 128) {
                    uint4 v[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        v[j] = m0 + j < p.M ? __ldg(reinterpret_cast<const uint4*>(p.x_raw + (size_t)(m0 + j) * p.K) + c)
                                            : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __bfloat1622float2(h[e]);
                            ss[j] = fmaf(f.x, f.x, ss[j]);
                            ss[j] = fmaf(f.y, f.y, ss[j]);
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    ss[j] = rv_warp_sum(ss[j]);
                    if (lane == 0 && m0 + j < p.M) norm_red[warp - 2][m0 + j] = ss[j];
                }
            }
            epi_sync();
            if (et < p.M)
                norm_rstd[et] = 1.0f / sqrtf((norm_red[0][et] + norm_red[1][et] + norm_red[2][et] + norm_red[3][et]) / (float)p.K + p.norm_eps);
            epi_sync();
            // ---- scale the activation tiles: thread = one 16-byte piece (row et / 8, piece et % 8 as
            // stored; the 128-byte swizzle put logical piece c at position c ^ (row % 8))
            const int row = et >> 3, pc = et & 7;
            const int lc = pc ^ (row & 7);
            const float r = row < p.M ? norm_rstd[row] : 0.f;
            int stage = 0;
            uint32_t phase = 0;
            for (int i = 0; i < n_kb; ++i) {
                const int kb = kb_at(i);
                float g[8];
                {
                    const float4 g0 = *reinterpret_cast<const float4*>(gam + (kb - kb0) * BK + lc * 8);
                    const float4 g1 = *reinterpret_cast<const float4*>(gam + (kb - kb0) * BK + lc * 8 + 4);
                    g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
                }
                // the whole warp leaves together, or a lane would wait in __syncwarp for ever
                if (!__all_sync(0xffffffffu, mbar_wait(full0 + 8 * stage, phase, &abort_flag, 5))) break;
                if (row < p.M) {
                    uint4* piece = reinterpret_cast<uint4*>(tiles + (size_t)stage * STAGE_BYTES + A_BYTES + row * 128 + pc * 16);
                    uint4 v = *piece;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __bfloat1622float2(h[e]);
                        h[e] = __floats2bfloat162_rn(f.x * r * g[2 * e], f.y * r * g[2 * e + 1]);
                    }
                    *piece = v;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(normed0 + 8 * stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
        // rows of the tile that this CTA finishes, and the bytes that all CTAs of the cluster (itself among them) send for them
        const int my_rows = p.cluster ? max(0, min(p.M, (split + 1) * p.cluster_rows) - split * p.cluster_rows) : 0;
        if (p.cluster) {
            cluster_wait();                                 // all CTAs of the cluster have started and set their barriers up
            if (et == 0 && my_rows > 0) mbar_expect_tx(xbar, (uint32_t)(p.splits * my_rows * TILE_F * 4));
        }
        if (have) mbar_wait(tfull, 0, &abort_flag, 4);
        // every epilogue thread comes here in bounded time; after the barrier they all see the same
        // abort flag, so the named barriers below are never reached by only some of them
        epi_sync();
        const bool ok = abort_flag == 0;
        tcgen05_fence_after();
        // [128 features][FS]: the stages are free now.  A feature's rows lie side by side and are moved four
        // at a time (16-byte accesses; with a stride of MB + 4 floats the eight lanes of a quarter warp
        // touch all 32 banks once), which also gives every thread four independent results to work on:
        // with one warp per scheduler the epilogue is bound by the latency of dependent instructions.
        constexpr int FS = MB + 4;
        float* fin = reinterpret_cast<float*>(tiles);
        if (ok) {
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            float* part = (p.splits > 1 && !p.cluster) ? p.scratch + ((size_t)(tile * p.splits + split) * MB) * TILE_F : nullptr;
            // One loop per destination (a branch per element costs more than the element does here).
            auto load16 = [&](int c, uint32_t (&r)[16]) {
                if (have) {
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                                 : "r"(taddr + c));
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int e = 0; e < 16; ++e) r[e] = 0u;    // this split got no k block: it adds zeros
                }
            };
            if (p.cluster) {
                // The partial goes row by row ([row][128 features] floats) into this CTA's shared memory, where its
                // stages were; the rows of CTA o (o * cluster_rows onwards) are one piece of it, which one bulk copy
                // takes to that CTA's buffer at [this split][its rows] and counts on its barrier.  (Stores into another
                // CTA's shared memory, one thread per feature and row, left an SM at about 20 GB/s.)
                float* stage_rows = reinterpret_cast<float*>(tiles);
#pragma unroll
                for (int c = 0; c < MB; c += 16) {
                    if (c >= p.M) break;
                    uint32_t r[16];
                    load16(c, r);
#pragma unroll
                    for (int e = 0; e < 16; ++e)
                        if (c + e < p.M) stage_rows[(c + e) * TILE_F + f] = __uint_as_float(r[e]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                epi_sync();
                if (et == 0) {
                    for (int o = 0; o < p.splits; ++o) {
                        const int r0 = o * p.cluster_rows, rows = min(p.M, r0 + p.cluster_rows) - r0;
                        if (rows <= 0) break;
                        bulk_copy_to_cluster(cluster_map(smem_u32(red) + (uint32_t)(split * p.cluster_rows * TILE_F) * 4u, (uint32_t)o),
                                             smem_u32(stage_rows) + (uint32_t)(r0 * TILE_F) * 4u, (uint32_t)(rows * TILE_F) * 4u,
                                             cluster_map(xbar, (uint32_t)o));
                    }
                    bulk_commit();
                }
            } else if (part) {
#pragma unroll
                for (int c = 0; c < MB; c += 16) {
                    if (c >= p.M) break;
                    uint32_t r[16];
                    load16(c, r);
#pragma unroll
                    for (int e = 0; e < 16; ++e)
                        if (c + e < p.M) part[(size_t)(c + e) * TILE_F + f] = __uint_as_float(r[e]);   // real rows only
                }
            } else {
#pragma unroll
                for (int c = 0; c < MB; c += 16) {
                    if (c >= p.M) break;                   // rows beyond M are never read below
                    uint32_t r[16];
                    load16(c, r);
                    float4* dst = reinterpret_cast<float4*>(fin + f * FS + c);
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        dst[e] = make_float4(__uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]),
                                             __uint_as_float(r[4 * e + 2]), __uint_as_float(r[4 * e + 3]));
                }
            }
            bool finish = true;
            if (p.splits > 1) {
                // Plain and rotary products: the partials are added and the epilogue is run in one
                // pass (finish_from_parts).  In a cluster every CTA does so for its rows, after the
                // cluster's barrier; else the CTA that arrives last at the tile's counter, for all rows.
                bool from_parts = false;
                const float* parts = nullptr;
                if (p.cluster) {
                    // every CTA's piece for this CTA's rows has arrived (a CTA without rows waits for nothing)
                    from_parts = my_rows > 0 && mbar_wait(xbar, 0, &abort_flag, 6);
                    parts = red;
                    finish = false;
                } else {
                    __threadfence();
                    epi_sync();
                    if (et == 0) is_last = atomicAdd(&p.counters[tile], 1) == p.splits - 1;
                    epi_sync();
                    finish = is_last != 0;
                    if (finish && !p.gated && (!p.q_out || p.hd >= 8)) {
                        __threadfence();
                        from_parts = true;
                        parts = p.scratch + ((size_t)tile * p.splits * MB) * TILE_F;
                        finish = false;                    // nothing is left for the shared epilogue below
                    }
                }
                if (from_parts) {
                    if (p.cluster) {
                        finish_from_parts<MB, true>(p, tile, et, parts, p.cluster_rows, split * p.cluster_rows,
                                                    min(p.M, (split + 1) * p.cluster_rows), row_pos, row_slot);
                    } else {
                        finish_from_parts<MB, false>(p, tile, et, parts, MB, 0, p.M, row_pos, row_slot);
                        if (et == 0) p.counters[tile] = 0;     // ready for the next launch
                    }
                }
                if (finish) {
                    __threadfence();
                    const float* base = p.scratch + ((size_t)tile * p.splits * MB) * TILE_F;
                    // the loads of four rows (up to 8 splits each) are in flight together; every row
                    // is summed in split order
                    for (int m0 = 0; m0 < p.M; m0 += 4) {
                        float v[4] = {0.f, 0.f, 0.f, 0.f};
                        for (int s0 = 0; s0 < p.splits; s0 += 8) {
                            float t[4][8];
#pragma unroll
                            for (int j = 0; j < 4; ++j)
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    t[j][i] = (m0 + j < p.M && s0 + i < p.splits)
                                                  ? __ldcg(base + ((size_t)(s0 + i) * MB + m0 + j) * TILE_F + f) : 0.f;
#pragma unroll
                            for (int j = 0; j < 4; ++j)
#pragma unroll
                                for (int i = 0; i < 8; ++i) v[j] += t[j][i];
                        }
                        *reinterpret_cast<float4*>(fin + f * FS + m0) = make_float4(v[0], v[1], v[2], v[3]);
                    }
                    if (et == 0) p.counters[tile] = 0;     // ready for the next launch
                }
            }
            if (finish) {
                epi_sync();
                if (p.gated) {
                    // features 0..63 are gate rows, 64..127 the up rows of the same output columns
                    const int fo = et & 63;
                    const int n = tile * (TILE_F / 2) + fo;
                    // eight rows of an output column per pass: eight independent chains per thread
                    for (int m0 = (et >> 6) * 8; m0 < p.M && n < half_n; m0 += 16) {
                        const float4 ga = *reinterpret_cast<const float4*>(fin + fo * FS + m0);
                        const float4 gb = *reinterpret_cast<const float4*>(fin + fo * FS + m0 + 4);
                        const float4 ua = *reinterpret_cast<const float4*>(fin + (fo + 64) * FS + m0);
                        const float4 ub = *reinterpret_cast<const float4*>(fin + (fo + 64) * FS + m0 + 4);
                        const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
                        const float u[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
                        float v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] = silu_gate(g[j], u[j], p.out_f32 != 0);
                        if (p.out_f32) {
                            float* o = (float*)p.out + (size_t)m0 * half_n + n;
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (m0 + j < p.M) o[(size_t)j * half_n] = v[j];
                        } else {
                            __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)m0 * half_n + n;
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (m0 + j < p.M) o[(size_t)j * half_n] = __float2bfloat16_rn(v[j]);
                        }
                    }
                } else if (p.q_out) {
                    // positions and slots of the rows once per CTA, then four rows at a time so that
                    // their table reads are in flight together
                    if (et < p.M) {
                        const int pos = p.positions[et];
                        row_pos[et] = pos < 0 ? 0 : (pos >= p.table_rows ? p.table_rows - 1 : pos);
                        row_slot[et] = p.slot_mapping[et];
                    }
                    epi_sync();
                    const int n = tile * TILE_F + et;
                    if (n < p.N) {
                        const int hd = p.hd, half = hd >> 1;
                        const int head = n / hd, d = n - head * hd;
                        const bool is_q = head < p.nh, is_k = !is_q && head < p.nh + p.nkv;
                        const bool rotate = (is_q || is_k) && p.cos_t != nullptr;
                        const bool first = d < half;
                        const int pe = first ? et + half : et - half;          // the pair's other feature
                        const int i = first ? d : d - half;
                        const float b = p.bias ? rv_load_param(p.bias, p.bias_dtype, n) : 0.f;
                        const float bp = p.bias ? rv_load_param(p.bias, p.bias_dtype, first ? n + half : n - half) : 0.f;
                        const int kvh = is_k ? head - p.nh : head - p.nh - p.nkv;
                        for (int m0 = 0; m0 < p.M; m0 += 4) {
                            float c[4], sn[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                c[j] = 1.f; sn[j] = 0.f;
                                if (rotate && m0 + j < p.M) {
                                    c[j] = __ldg(p.cos_t + (size_t)row_pos[m0 + j] * half + i);
                                    sn[j] = __ldg(p.sin_t + (size_t)row_pos[m0 + j] * half + i);
                                }
                            }
                            const float4 own4 = *reinterpret_cast<const float4*>(fin + et * FS + m0);
                            const float4 other4 = *reinterpret_cast<const float4*>(fin + pe * FS + m0);
                            const float owns[4] = {own4.x, own4.y, own4.z, own4.w}, others[4] = {other4.x, other4.y, other4.z, other4.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int m = m0 + j;
                                if (m >= p.M) break;
                                const float own = owns[j] + b;
                                float v = own;
                                if (is_q || is_k) {
                                    const float other = others[j] + bp;
                                    v = first ? own * c[j] - other * sn[j] : other * sn[j] + own * c[j];
                                }
                                if (is_q) {
                                    p.q_out[(size_t)m * p.nh * hd + n] = __float2bfloat16_rn(v);
                                } else {
                                    const int slot = row_slot[m];
                                    if (slot >= 0) {
                                        const int page = slot / p.page_size, off = slot - page * p.page_size;
                                        p.kv_cache[((((size_t)page * 2 + (is_k ? 0 : 1)) * p.nkv + kvh) * p.page_size + off) * hd + d] =
                                            __float2bfloat16_rn(v);
                                    }
                                }
                            }
                        }
                    }
                } else {
                    const int n = tile * TILE_F + et;
                    if (n < p.N) {
                        const float b = p.bias ? rv_load_param(p.bias, p.bias_dtype, n) : 0.f;
                        for (int m0 = 0; m0 < p.M; m0 += 8) {
                            float r8[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                r8[j] = (p.residual && m0 + j < p.M) ? __bfloat162float(p.residual[(size_t)(m0 + j) * p.N + n]) : 0.f;
                            const float4 lo4 = *reinterpret_cast<const float4*>(fin + et * FS + m0);
                            const float4 hi4 = *reinterpret_cast<const float4*>(fin + et * FS + m0 + 4);
                            const float acc8[8] = {lo4.x, lo4.y, lo4.z, lo4.w, hi4.x, hi4.y, hi4.z, hi4.w};
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const int m = m0 + j;
                                if (m >= p.M) break;
                                const float v = acc8[j] + b + r8[j];
                                if (p.out_f32) ((float*)p.out)[(size_t)m * p.N + n] = v;
                                else ((__nv_bfloat16*)p.out)[(size_t)m * p.N + n] = __float2bfloat16_rn(v);
                            }
                        }
                    }
                }
            }
        } else if (p.cluster && my_rows > 0) {
            // gave up: what the other CTAs send still lands in this CTA's shared memory, which must not be given up before
            volatile int ignore = 0;
            mbar_wait(xbar, 0, &ignore, 0);
        }
        if (p.cluster && et == 0) bulk_wait_read();         // the copies have read this CTA's rows: its shared memory may go
    }

    // The cluster's barrier has one phase (every CTA runs and has set its barriers up): the epilogue warps waited for it
    // before they sent anything, warps 0 and 1 do so at the very end.  The hand-over of the partials is counted on
    // the receiving CTA's own barrier.
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
    if (threadIdx.x == 0 && abort_flag != 0 && p.status) atomicCAS(p.status, 0, abort_flag);
    if (p.cluster && warp < 2) cluster_wait();
}

template <int MB>
static int launch_decode(const CUtensorMap& mw, const CUtensorMap& mx, const DecodeGemmParams& p, cudaStream_t stream) {
    constexpr int STAGES = STAGES_FOR(MB);
    const int stage = A_BYTES + MB * BK * 2;
    const int fin = TILE_F * (MB + 4) * 4;
    int smem = (STAGES * stage > fin ? STAGES * stage : fin) + 1024;
    static RvPerDevice configured;
    if (int e = rv_configure_smem(configured, gemm_decode_kernel<MB>, smem + MAX_NORM_K * 4 + (64 + 8) * TILE_F * 4)) return e;
    if (p.norm_gamma || p.cluster) {
        const int num_kb = (p.K + BK - 1) / BK;
        smem = STAGES * stage + 1024;
        if (p.norm_gamma) smem += ((num_kb + p.splits - 1) / p.splits) * BK * 4;     // gamma of a CTA's K range behind the stages
        if (p.cluster) smem += p.splits * p.cluster_rows * TILE_F * 4;              // the partials of this CTA's rows behind that
        if (smem < fin + 1024) smem = fin + 1024;
    }
    const int row_blocks = MB == 128 ? (p.M + MB - 1) / MB : 1;
    if (p.cluster)
        RV_LAUNCH_ST = rv_launch_cluster(gemm_decode_kernel<MB>, dim3(p.n_tiles * p.splits, row_blocks), dim3(NUM_THREADS), smem, stream,
                                         (unsigned)p.splits, mw, mx, p);
    else
        RV_LAUNCH_ST = rv_launch(gemm_decode_kernel<MB>, dim3(p.n_tiles * p.splits, row_blocks), dim3(NUM_THREADS), smem, stream, mw, mx, p);
    return rv_launch_status();
}

// Rows of batch padding this kernel would use for M rows (16, 32, 64 or 128).
RV_EXPORT int rv_gemm_decode_padded_rows(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128)); }

// Number of 128-feature tiles, so that the caller can size `scratch` (tiles * splits * padded rows
// * 128 floats when splits > 1) and `counters` (tiles ints, zero before the first launch; the
// kernel leaves them zero).
RV_EXPORT int rv_gemm_decode_tiles(int N, int gated) {
    return gated ? (N / 2 + TILE_F / 2 - 1) / (TILE_F / 2) : (N + TILE_F - 1) / TILE_F;
}

static int g_l2_ahead = 0;
static int g_k_rotate = 0;
// The K loop of tile t starts at k block (t * step) mod the CTA's count (0: every tile at its first block).
RV_EXPORT void rv_gemm_decode_set_k_rotate(int step) { g_k_rotate = step < 0 ? 0 : step; }
// How many k blocks of weights beyond its shared-memory stages a CTA asks into L2 before it waits for
// the previous kernel (0: none).
RV_EXPORT void rv_gemm_decode_set_l2_ahead(int k_blocks) { g_l2_ahead = k_blocks < 0 ? 0 : k_blocks; }

static int run_decode(const void* x, const void* w, DecodeGemmParams p, cudaStream_t stream) {
    p.l2_ahead = g_l2_ahead;
    p.k_rotate = g_k_rotate;
    if (p.M < 0 || p.N <= 0 || p.K <= 0 || p.splits < 1) return RV_ERR_BAD_SIZE;
    if (p.M > 128 * 512) return RV_ERR_UNSUPPORTED;
    // blocks of 128 rows share neither scratch nor counters: beyond 128 rows K is split inside a cluster, or not at all
    if (p.M > 128 && p.splits > 1 && !(p.cluster && p.splits <= 8 && !p.gated && (!p.q_out || p.hd >= 8))) return RV_ERR_UNSUPPORTED;
    if (p.K % 8) return RV_ERR_UNSUPPORTED;
    if (p.norm_gamma && p.M > 16) return RV_ERR_UNSUPPORTED;       // the fused norm serves one 16-row tile
    if (p.norm_gamma && (p.K + BK - 1) / BK * BK > MAX_NORM_K) return RV_ERR_UNSUPPORTED;
    p.x_raw = (const __nv_bfloat16*)x;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16) return RV_ERR_ALIGNMENT;
    if (p.M == 0) return RV_OK;
    const int num_kb = (p.K + BK - 1) / BK;
    if (p.splits > num_kb) p.splits = num_kb;
    // few rows, few splits, an epilogue that adds partials four features at a time: the CTAs of a tile
    // form a cluster and add up in shared memory
    p.cluster = (p.cluster && p.splits >= 2 && p.splits <= 8 && !p.gated && (!p.q_out || p.hd >= 8)) ? 1 : 0;
    p.cluster_rows = ((p.M < 128 ? p.M : 128) + p.splits - 1) / p.splits;
    if (p.splits > 1 && !p.cluster && (!p.scratch || !p.counters)) return RV_ERR_BAD_SIZE;
    const int mb = rv_gemm_decode_padded_rows(p.M);
    alignas(64) CUtensorMap mw, mx;
    int st = rv_make_bf16_map(&mw, w, p.N, p.K, TILE_F / 2);
    if (st != RV_OK) return st;
    st = rv_make_bf16_map(&mx, x, p.M, p.K, mb);
    if (st != RV_OK) return st;
    p.n_tiles = rv_gemm_decode_tiles(p.N, p.gated);
    switch (mb) {
        case 16: return launch_decode<16>(mw, mx, p, stream);
        case 32: return launch_decode<32>(mw, mx, p, stream);
        case 64: return launch_decode<64>(mw, mx, p, stream);
        default: return launch_decode<128>(mw, mx, p, stream);
    }
}

RV_EXPORT int rv_gemm_tcgen05_decode_bf16(const void* x, const void* w, const void* bias, int bias_dtype,
                                          const void* residual, void* out, int out_f32, int M, int N, int K,
                                          int gated, int splits, int cluster, float* scratch, int* counters, int* status,
                                          const void* norm_gamma, int norm_gamma_dtype, float norm_eps,
                                          cudaStream_t stream) {
    if (gated && ((N & 1) || bias || residual)) return RV_ERR_BAD_SIZE;
    if (residual && out_f32) return RV_ERR_BAD_SIZE;
    DecodeGemmParams p = {};
    p.out = out; p.residual = (const __nv_bfloat16*)residual; p.bias = bias; p.bias_dtype = bias_dtype;
    p.scratch = scratch; p.counters = counters; p.status = status;
    p.M = M; p.N = N; p.K = K; p.out_f32 = out_f32; p.gated = gated; p.splits = splits; p.cluster = cluster;
    p.norm_gamma = norm_gamma; p.norm_gamma_dtype = norm_gamma_dtype; p.norm_eps = norm_eps;
    return run_decode(x, w, p, stream);
}

// cluster (both entry points): 1 asks for the reduction inside a thread-block cluster where the
// kernel can do it (2 to 8 splits, up to 64 rows, not gated); scratch and counters are then unused.
// norm_gamma (both entry points): RMSNorm weights [K] applied to x inside the kernel (M <= 16), or nullptr.
// The q/k/v product of an attention layer with bias, rotation and the cache write in its epilogue.
// w: [(nh + 2 nkv) * hd, K]; q_out: [M, nh * hd]; kv_cache: [pages, 2, nkv, page_size, hd].
RV_EXPORT int rv_gemm_decode_qkv_rope(const void* x, const void* w, const void* bias, int bias_dtype,
                                      const int* positions, const float* cos_t, const float* sin_t,
                                      const int* slot_mapping, void* kv_cache, void* q_out, int M, int K,
                                      int nh, int nkv, int hd, int page_size, int table_rows, int splits, int cluster,
                                      float* scratch, int* counters, int* status, const void* norm_gamma,
                                      int norm_gamma_dtype, float norm_eps, cudaStream_t stream) {
    if (nh <= 0 || nkv <= 0 || hd <= 0 || (hd & 1) || page_size <= 0 || table_rows <= 0) return RV_ERR_BAD_SIZE;
    if (TILE_F % hd) return RV_ERR_UNSUPPORTED;           // a rotation pair must lie in one tile
    if ((cos_t == nullptr) != (sin_t == nullptr)) return RV_ERR_BAD_SIZE;
    if (!positions || !slot_mapping || !kv_cache || !q_out) return RV_ERR_BAD_SIZE;
    DecodeGemmParams p = {};
    p.bias = bias; p.bias_dtype = bias_dtype;
    p.scratch = scratch; p.counters = counters; p.status = status;
    p.M = M; p.N = (nh + 2 * nkv) * hd; p.K = K; p.splits = splits; p.cluster = cluster;
    p.q_out = (__nv_bfloat16*)q_out; p.kv_cache = (__nv_bfloat16*)kv_cache; p.positions = positions;
    p.slot_mapping = slot_mapping; p.cos_t = cos_t; p.sin_t = sin_t;
    p.nh = nh; p.nkv = nkv; p.hd = hd; p.page_size = page_size; p.table_rows = table_rows;
    p.norm_gamma = norm_gamma; p.norm_gamma_dtype = norm_gamma_dtype; p.norm_eps = norm_eps;
    return run_decode(x, w, p, stream);
}
