// bfloat16 linear layer on the fifth-generation tensor cores of sm_100a:
//     out[M, N] = x[M, K] . W[N, K]^T  (+ residual[M, N]),  float accumulate, bf16 or float out,
// or, GATED, with W rows [gate (N/2) | up (N/2)]:  out[M, N/2] = silu(x Wg^T) * (x Wu^T).
//
// Structure (one CTA per SM, persistent over output tiles of 128 x 256):
//   warp 0   TMA producer: cp.async.bulk.tensor loads of a 128 x 64 tile of x and a 256 x 64 tile
//            of W per stage (128-byte swizzle), 4 stages, completion on mbarriers;
//   warp 1   MMA issuer: one elected thread issues tcgen05.mma (M = 128, N = 256, K = 16, both
//            operands K-major from shared memory, accumulator in tensor memory); tcgen05.commit
//            frees a stage for the producer and, after the last k block, hands the accumulator to
//            the epilogue.  Two accumulators (2 x 256 TMEM columns) let tile i+1 start while
//            tile i is written out;
//   warps 2-5  epilogue: tcgen05.ld 32 lanes x 32 columns at a time, add the residual / apply
//            SiLU-gate in float, round once, store.  For the q/k/v product of an attention layer
//            the epilogue rounds the sums as a separate product would store them, adds the bias,
//            rotates q and k by the row's position (a head's two halves are read from tensor memory
//            side by side), writes q to its output and k and v straight into the row's slot of the
//            paged cache: the rotary kernel and the round trip of q/k/v through memory are saved.
// No multicast load.  Every wait on an mbarrier is bounded: when a wait gives up, the CTA
// sets an abort flag, every role leaves its loop, the producer waits (bounded) for its loads in
// flight, tensor memory is freed, the kernel writes a status word and returns.
//
// Compiled with -DRV_PAIR=1 the same source is the kernel on PAIRS of CTAs (tcgen05 cta_group::2).  Two
// CTAs on neighbouring SMs (a thread-block cluster of 2) own one output tile of 256 x 256.  Each CTA
// fetches its own 128 rows of x and only HALF of the tile's 256 weight rows (32 KB per stage instead of
// 48 KB, six stages instead of four); the first CTA of the pair issues tcgen05.mma.cta_group::2, which
// reads the two halves of the weights from the two CTAs' shared memory and accumulates 128 rows x 256
// columns in each CTA's tensor memory.  Both CTAs' loads are counted on the first CTA's mbarrier;
// tcgen05.commit with multicast frees a stage in both CTAs and hands the accumulator to both CTAs'
// epilogue warps, which arrive on the first CTA's barrier when they have read it out; the pair leaves
// together through a cluster barrier.  Why it is faster: with one CTA a k block takes (load latency +
// MMA time) / 4 stages, because four stages of 48 KB are all that fit, and 128 x 256 x 64 MACs per
// 0.39 us ask for 123 GB/s per SM with about 1.2 us of latency; 32 KB per k block need 98 KB in flight.
// The epilogues and the sums are the same in both builds (same bits).
//
// Shapes: the five products of a layer at prefill time
// (v3/crates/rvllm-runtime/src/layer_exec.rs:240-266,433-444,478-488,511-522 of the reference,
// which calls cuBLASLt; its residual epilogue beta = 1 is cublaslt.rs:335-368, and its fused
// gate-up-SiLU idea is kernels/cutlass_gateup_silu.cu).
#include "common.cuh"
#include "tcgen05.cuh"

#ifndef RV_PAIR
#define RV_PAIR 0
#endif
#define BM 128
#ifndef BN
#define BN 256          // columns of an output tile; -DBN=128 builds the narrow tiles for products that would not fill the SMs
#endif
static_assert(BN == 256 || BN == 128, "tiles of 256 or 128 columns");
#define BK 64
#define UMMA_K 16
#define A_TILE_BYTES (BM * BK * 2)
#if RV_PAIR
#define STAGES 6
#define TILE_ROWS (2 * BM)                      // rows of an output tile: both CTAs' 128
#define B_TILE_BYTES (BN / 2 * BK * 2)          // this CTA's half of the tile's weight rows
#define CTA_GROUP "2"
#define gemm_tcgen05_kernel gemm_tcgen05_pair_kernel
#else
#define STAGES 4
#define TILE_ROWS BM
#define B_TILE_BYTES (BN * BK * 2)
#define CTA_GROUP "1"
#endif
#define STAGE_BYTES (A_TILE_BYTES + B_TILE_BYTES)
#define NUM_THREADS 192
#define TMEM_COLS 512

#define EPI_PLAIN 0
#define EPI_RESIDUAL 1
#define EPI_GATED 2
#define EPI_ROPE 3          // the q/k/v product: bias, rotation of q and k, k and v into the paged cache

struct GemmParams {
    void* out;
    const __nv_bfloat16* residual;
    int* status;            // device word: 0 ok, else the code of the wait that gave up
    int M, N, K;
    int out_f32;
    int epilogue;
    int m_tiles, n_tiles;   // tiles of TILE_ROWS rows x BN columns
    // K cut into `splits` parts (1, 2 or 4; the build on single CTAs only): the CTAs of a tile are a thread-block
    // cluster, every CTA keeps BN / splits columns of the tile, gets the other CTAs' partials of those columns into
    // its shared memory (where its stages were) and adds them in the order of the parts.  Not for EPI_GATED.
    int splits;
    // EPI_ROPE: W rows are [q heads | k heads | v heads] of hd (64, 128 or 256) features
    const void* bias;                // [N] or nullptr
    int bias_dtype;
    __nv_bfloat16* q_out;            // [M, nh * hd]
    __nv_bfloat16* kv_cache;         // [pages, 2, nkv, page_size, hd]
    const int* positions;            // [M]
    const int* slot_mapping;         // [M], < 0: the row writes no key or value
    const float* cos_t;              // [table_rows, hd / 2] or nullptr (no rotation)
    const float* sin_t;
    int nh, nkv, hd, page_size, table_rows;
};


__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }
// a cluster of CTAs that share a tile's K (the build on single CTAs)
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }     // the four epilogue warps
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// One bulk copy from this CTA's shared memory into another CTA's of the cluster; its bytes are counted on a barrier
// of the receiving CTA (both given as addresses in the cluster's shared window).
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t dst, uint32_t src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "r"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// EPI_ROPE: columns d .. d + 31 (a) and d + hd/2 .. d + hd/2 + 31 (b) of one head of row m.
__device__ __forceinline__ void store_rope_pair(const GemmParams& p, int m, int head, int d, const uint32_t (&ra)[32],
                                                const uint32_t (&rb)[32], int pos, int slot) {
    const int hd = p.hd, half = hd >> 1;
    const bool is_q = head < p.nh, is_k = !is_q && head < p.nh + p.nkv;
    const int n_a = head * hd + d, n_b = n_a + half;
    __nv_bfloat16 *dst_a, *dst_b;
    if (is_q) {
        dst_a = p.q_out + (size_t)m * p.nh * hd + n_a;
    } else {
        if (slot < 0) return;
        const int kvh = is_k ? head - p.nh : head - p.nh - p.nkv;
        const int page = slot / p.page_size, off = slot - page * p.page_size;
        dst_a = p.kv_cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * p.nkv + kvh) * p.page_size + off) * hd + d;
    }
    dst_b = dst_a + half;
    const bool rotate = (is_q || is_k) && p.cos_t != nullptr;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        float c[8], sn[8];
        if (rotate) {
            const float4* cp = reinterpret_cast<const float4*>(p.cos_t + (size_t)pos * half + d + v * 8);
            const float4* sp = reinterpret_cast<const float4*>(p.sin_t + (size_t)pos * half + d + v * 8);
            const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
            c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
            sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
        }
        uint4 oa, ob;
        __nv_bfloat16* oae = reinterpret_cast<__nv_bfloat16*>(&oa);
        __nv_bfloat16* obe = reinterpret_cast<__nv_bfloat16*>(&ob);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int e = v * 8 + j;
            // the float accumulators go into bias and rotation as they are: one rounding, at the store
            float a = __uint_as_float(ra[e]);
            float b = __uint_as_float(rb[e]);
            if (p.bias) {
                a += rv_load_param(p.bias, p.bias_dtype, n_a + e);
                b += rv_load_param(p.bias, p.bias_dtype, n_b + e);
            }
            if (rotate) {
                oae[j] = __float2bfloat16_rn(a * c[j] - b * sn[j]);
                obe[j] = __float2bfloat16_rn(a * sn[j] + b * c[j]);
            } else {
                oae[j] = __float2bfloat16_rn(a);
                obe[j] = __float2bfloat16_rn(b);
            }
        }
        *reinterpret_cast<uint4*>(dst_a + v * 8) = oa;
        *reinterpret_cast<uint4*>(dst_b + v * 8) = ob;
    }
}

// ---- a pair of CTAs (RV_PAIR): addresses in the other CTA, loads and commits that signal across the pair
__device__ __forceinline__ uint32_t pair_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t pair_map(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// TMA tile load into this CTA's shared memory whose bytes are counted on `bar`, a barrier of either CTA
// of the pair (an address in the cluster's shared window)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16_pair(uint32_t tmem_c, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                      uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_c), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive on the barrier at this shared-memory offset in BOTH CTAs once the MMAs issued so far are done
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void pair_sync() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// the MMA and the commit of this build
__device__ __forceinline__ void mma_issue(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    if (RV_PAIR) tcgen05_mma_bf16_pair(tmem_c, da, db, idesc, accumulate);
    else tcgen05_mma_bf16(tmem_c, da, db, idesc, accumulate);
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    if (RV_PAIR) tcgen05_commit_pair(bar);
    else tcgen05_commit(bar);
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 5];     // full, empty, accumulator full / empty [2], partials arrived
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    rv_pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t tfull0 = smem_u32(&bars[2 * STAGES]), tempty0 = smem_u32(&bars[2 * STAGES + 2]);
    const uint32_t xbar = smem_u32(&bars[2 * STAGES + 4]);     // K over a cluster: the other CTAs' partials of this CTA's columns

    // pair: rank 0 issues the MMAs and owns the barriers that count both CTAs (full, tempty)
    const uint32_t rank = RV_PAIR ? pair_rank() : 0u;
    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&map_a);
        tma_prefetch_descriptor(&map_b);
        abort_flag = 0;
        // full: one arrival (the producer; in a pair the first CTA's, with the bytes of both CTAs);
        // empty, tfull: one arrival from the commit; tempty: the four epilogue warps (of both CTAs)
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, RV_PAIR ? 8 : 4); }
        mbar_init(xbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // (with cta_group::2 one warp of each CTA of the pair executes the allocation; both get the same address)
        asm volatile("tcgen05.alloc.cta_group::" CTA_GROUP ".sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::" CTA_GROUP ".sync.aligned;" ::);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    if (RV_PAIR) pair_sync();       // both CTAs' barriers exist before either signals the other's
    rv_pdl_wait();          // the set-up above overlapped the previous kernel; its results are needed from here

    const int num_tiles = p.m_tiles * p.n_tiles;
    // the persistent workers: CTAs, or pairs of CTAs
    const int S = (!RV_PAIR && p.splits > 1) ? p.splits : 1;          // CTAs of a cluster that share a tile's K
    const int split = S > 1 ? (int)blockIdx.x % S : 0;                 // (the rank in the cluster)
    const int worker = RV_PAIR ? blockIdx.x >> 1 : blockIdx.x / S, num_workers = RV_PAIR ? gridDim.x >> 1 : gridDim.x / S;
    const int num_kb = (p.K + BK - 1) / BK;
    const int kb_per = (num_kb + S - 1) / S;
    const int kb_first = split * kb_per, kb_last = min(num_kb, kb_first + kb_per);     // this CTA's k blocks
    const bool gated = p.epilogue == EPI_GATED;
    const int half_n = p.N >> 1;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int issued = 0;
            bool ok = true;
            for (int tile = worker; tile < num_tiles && ok; tile += num_workers) {
                const int m0 = (tile % p.m_tiles) * TILE_ROWS + (int)rank * BM;      // this CTA's 128 rows
                const int nt = tile / p.m_tiles;
                for (int kb = kb_first; kb < kb_last; ++kb) {
                    if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, &abort_flag, 1)) { ok = false; break; }
                    const uint32_t a_dst = smem_u32(tiles + (size_t)stage * STAGE_BYTES);
                    const uint32_t b_dst = a_dst + A_TILE_BYTES;
                    if (RV_PAIR) {
                        // this CTA's 128 of the tile's 256 weight rows (gated: the first CTA has the gate
                        // rows, the second the up rows of the same output columns); the first CTA's
                        // barrier counts both CTAs' bytes
                        const int w0 = gated ? (rank == 0 ? nt * (BN / 2) : half_n + nt * (BN / 2)) : nt * BN + (int)rank * (BN / 2);
                        const uint32_t bar = pair_map(full0 + 8 * stage, 0);
                        if (rank == 0) mbar_expect_tx(full0 + 8 * stage, 2 * STAGE_BYTES);
                        tma_load_2d_pair(a_dst, &map_a, kb * BK, m0, bar);
                        tma_load_2d_pair(b_dst, &map_b, kb * BK, w0, bar);
                        ++issued;
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                        continue;
                    }
                    const uint32_t bar = full0 + 8 * stage;
                    mbar_expect_tx(bar, STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, kb * BK, m0, bar);
                    if (gated) {       // 128 gate rows, then the 128 up rows of the same columns
                        tma_load_2d(b_dst, &map_b, kb * BK, nt * (BN / 2), bar);
                        tma_load_2d(b_dst + B_TILE_BYTES / 2, &map_b, kb * BK, half_n + nt * (BN / 2), bar);
                    } else {
                        tma_load_2d(b_dst, &map_b, kb * BK, nt * BN, bar);
                        tma_load_2d(b_dst + B_TILE_BYTES / 2, &map_b, kb * BK, nt * BN + BN / 2, bar);
                    }
                    ++issued;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // gave up: let the loads in flight land before the CTA's shared memory goes away
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
        // (the producer's and the issuer's warps take part in the cluster's barrier after their work)
        if (S > 1) { cluster_arrive(); cluster_wait(); }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = umma_idesc_bf16(TILE_ROWS, BN);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int tile = worker; tile < num_tiles && ok; tile += num_workers, ++local) {
                const int buf = local & 1;
                const uint32_t use = (uint32_t)(local >> 1);
                if (!mbar_wait(tempty0 + 8 * buf, (use & 1) ^ 1, &abort_flag, 2)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t tmem_c = tmem_base + (uint32_t)buf * BN;
                for (int kb = kb_first; kb < kb_last; ++kb) {
                    if (!mbar_wait(full0 + 8 * stage, phase, &abort_flag, 3)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + (size_t)stage * STAGE_BYTES);
                    const uint64_t da = umma_desc(a_addr), db = umma_desc(a_addr + A_TILE_BYTES);
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j) {
                        // 16 k = 32 bytes further along the 128-byte row: +2 in 16-byte units
                        mma_issue(tmem_c, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc, kb > kb_first || j != 0);
                    }
                    mma_commit(empty0 + 8 * stage);         // the stage is free (in both CTAs) once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) mma_commit(tfull0 + 8 * buf);       // accumulator complete (in both CTAs)
            }
        }
        if (S > 1) { cluster_arrive(); cluster_wait(); }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;                       // the TMEM lanes this warp may read
        int local = 0;
        bool ok = true;
        for (int tile = worker; tile < num_tiles && ok; tile += num_workers, ++local) {
            const int buf = local & 1;
            const uint32_t use = (uint32_t)(local >> 1);
            if (!mbar_wait(tfull0 + 8 * buf, use & 1, &abort_flag, 4)) {
                ok = false;
                if (S > 1) {     // the others still count on the barrier, and send what this CTA's shared memory has to outlive
                    if (warp == 2 && lane == 0) mbar_expect_tx(xbar, (uint32_t)(S - 1) * (uint32_t)(BM * (BN / S + 4)) * 4u);
                    cluster_arrive();
                    cluster_wait();
                    volatile int ignore = 0;
                    mbar_wait(xbar, 0, &ignore, 0);
                }
                break;
            }
            tcgen05_fence_after();
            const int m = (tile % p.m_tiles) * TILE_ROWS + (int)rank * BM + quarter * 32 + lane;
            const int nt = tile / p.m_tiles;
            const uint32_t taddr = tmem_base + (uint32_t)buf * BN + ((uint32_t)(quarter * 32) << 16);
            // ---- K in parts over a cluster: every CTA keeps cols_per columns of the tile.  After the cluster's barrier
            // (every CTA's products are done, so its stages are free) each thread writes its row's partial of the OTHER
            // CTAs' columns into this CTA's shared memory, one piece of [128 rows][cols_per + 4] floats per receiving
            // CTA, and one bulk copy per piece takes it into that CTA's shared memory, counted on that CTA's barrier.
            // Then the parts of the CTA's own columns are added in the order of the parts, its own from tensor memory.
            // (Per-row stores straight into the other CTAs' shared memory left an SM at 15 GB/s: 6.4 us for this.)
            const int cols_per = BN / S, RS = cols_per + 4;
            const int c_begin = S > 1 ? split * cols_per : 0, c_end = S > 1 ? c_begin + cols_per : BN;
            const uint32_t piece_bytes = (uint32_t)(BM * RS) * 4u;
            // [0, S - 1): pieces received (from part sp, at index sp or sp - 1 past this CTA); [S - 1, 2 S - 2): pieces to send
            float* pieces = reinterpret_cast<float*>(tiles);
            if (S > 1) {
                if (warp == 2 && lane == 0) mbar_expect_tx(xbar, (uint32_t)(S - 1) * piece_bytes);
                cluster_arrive();
                cluster_wait();
                if (abort_flag == 0) {
                    for (int c = 0; c < BN; c += 32) {
                        const int owner = c / cols_per;
                        if (owner == split) continue;
                        uint32_t r[32];
                        if (kb_first < kb_last) {
                            tmem_ld_32x32(taddr + c, r);
                            tmem_ld_wait();
                        } else {
#pragma unroll
                            for (int e = 0; e < 32; ++e) r[e] = 0u;        // a part without a k block (a short K) adds zeros
                        }
                        const int slot = S - 1 + (owner < split ? owner : owner - 1);
                        float4* dst = reinterpret_cast<float4*>(pieces + ((size_t)slot * BM + quarter * 32 + lane) * RS + (c - owner * cols_per));
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            dst[v] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                 __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    epi_sync();
                    if (warp == 2 && lane == 0) {
                        for (int owner = 0; owner < S; ++owner) {
                            if (owner == split) continue;
                            const int slot = S - 1 + (owner < split ? owner : owner - 1);     // here
                            const int there = split < owner ? split : split - 1;              // this part's place in the receiving CTA
                            bulk_copy_to_cluster(cluster_map(smem_u32(pieces) + (uint32_t)there * piece_bytes, (uint32_t)owner),
                                                 smem_u32(pieces) + (uint32_t)slot * piece_bytes, piece_bytes, cluster_map(xbar, (uint32_t)owner));
                        }
                        bulk_commit();
                    }
                }
                // the other parts' pieces have arrived (bounded; after a wait that gave up the flag says so)
                mbar_wait(xbar, 0, &abort_flag, 5);
            }
            // 32 accumulator columns of this thread's row: from tensor memory, or the parts' partials added in part order
            auto load_acc = [&](int col, uint32_t (&r)[32]) {
                tmem_ld_32x32(taddr + col, r);
                tmem_ld_wait();
                if (S == 1) return;
                if (kb_first >= kb_last) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) r[e] = 0u;
                }
                float acc[32];
                for (int sp = 0; sp < S; ++sp) {
                    if (sp == split) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) acc[e] = sp == 0 ? __uint_as_float(r[e]) : acc[e] + __uint_as_float(r[e]);
                        continue;
                    }
                    const int slot = sp < split ? sp : sp - 1;
                    const float4* src = reinterpret_cast<const float4*>(pieces + ((size_t)slot * BM + quarter * 32 + lane) * RS + (col - c_begin));
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const float4 t = src[v];
                        if (sp == 0) { acc[4 * v] = t.x; acc[4 * v + 1] = t.y; acc[4 * v + 2] = t.z; acc[4 * v + 3] = t.w; }
                        else { acc[4 * v] += t.x; acc[4 * v + 1] += t.y; acc[4 * v + 2] += t.z; acc[4 * v + 3] += t.w; }
                    }
                }
#pragma unroll
                for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(acc[e]);
            };
            if (gated) {
                const int n_out0 = nt * (BN / 2);
                for (int c = 0; c < BN / 2; c += 32) {
                    uint32_t g[32], u[32];
                    tmem_ld_32x32(taddr + c, g);
                    tmem_ld_32x32(taddr + BN / 2 + c, u);
                    tmem_ld_wait();
                    if (m < p.M) {
                        const int n = n_out0 + c;
                        if (!p.out_f32 && n + 32 <= half_n && (half_n & 7) == 0) {
                            __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (size_t)m * half_n + n;
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                uint4 o;
                                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const int e = v * 8 + 2 * j;
                                    oh[j] = __floats2bfloat162_rn(silu_f(__uint_as_float(g[e])) * __uint_as_float(u[e]),
                                                                  silu_f(__uint_as_float(g[e + 1])) * __uint_as_float(u[e + 1]));
                                }
                                *reinterpret_cast<uint4*>(dst + v * 8) = o;
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 32; ++e) {
                                if (n + e >= half_n) continue;
                                const float val = silu_f(__uint_as_float(g[e])) * __uint_as_float(u[e]);
                                if (p.out_f32) ((float*)p.out)[(size_t)m * half_n + n + e] = val;
                                else ((__nv_bfloat16*)p.out)[(size_t)m * half_n + n + e] = __float2bfloat16_rn(val);
                            }
                        }
                    }
                }
            } else if (p.epilogue == EPI_ROPE) {
                const int n0 = nt * BN;
                const int half = p.hd >> 1;
                int pos = 0, slot = -1;
                if (m < p.M) {
                    pos = p.positions[m];
                    pos = pos < 0 ? 0 : (pos >= p.table_rows ? p.table_rows - 1 : pos);
                    slot = p.slot_mapping[m];
                }
                for (int hb = c_begin; hb < c_end; hb += p.hd) {   // the heads of this tile (of this CTA's columns of it)
                    if (n0 + hb >= p.N) break;                      // uniform over the warp
                    const int head = (n0 + hb) / p.hd;
                    for (int c = 0; c < half; c += 32) {
                        uint32_t ra[32], rb[32];
                        load_acc(hb + c, ra);
                        load_acc(hb + half + c, rb);
                        if (m < p.M) store_rope_pair(p, m, head, c, ra, rb, pos, slot);
                    }
                }
            } else {
                const int n0 = nt * BN;
                for (int c = c_begin; c < c_end; c += 32) {
                    if (n0 + c >= p.N) break;              // uniform over the warp
                    uint32_t r[32];
                    load_acc(c, r);
                    if (m < p.M) {
                        const int n = n0 + c;
                        const bool vec = n + 32 <= p.N && (p.N & 7) == 0;
                        if (vec && !p.out_f32) {
                            __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (size_t)m * p.N + n;
                            const __nv_bfloat16* res = p.residual ? p.residual + (size_t)m * p.N + n : nullptr;
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                uint4 rv = make_uint4(0, 0, 0, 0);
                                if (res) rv = *reinterpret_cast<const uint4*>(res + v * 8);
                                const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&rv);
                                uint4 o;
                                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const int e = v * 8 + 2 * j;
                                    const float2 rf = __bfloat1622float2(rh[j]);
                                    oh[j] = __floats2bfloat162_rn(__uint_as_float(r[e]) + rf.x, __uint_as_float(r[e + 1]) + rf.y);
                                }
                                *reinterpret_cast<uint4*>(dst + v * 8) = o;
                            }
                        } else if (vec && p.out_f32 && !p.residual && (p.N & 3) == 0) {
                            float4* dst = reinterpret_cast<float4*>((float*)p.out + (size_t)m * p.N + n);
#pragma unroll
                            for (int v = 0; v < 8; ++v)
                                dst[v] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                     __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                        } else {
#pragma unroll
                            for (int e = 0; e < 32; ++e) {
                                if (n + e >= p.N) continue;
                                float val = __uint_as_float(r[e]);
                                if (p.residual) val += __bfloat162float(p.residual[(size_t)m * p.N + n + e]);
                                if (p.out_f32) ((float*)p.out)[(size_t)m * p.N + n + e] = val;
                                else ((__nv_bfloat16*)p.out)[(size_t)m * p.N + n + e] = __float2bfloat16_rn(val);
                            }
                        }
                    }
                }
            }
            if (S > 1 && warp == 2 && lane == 0) bulk_wait_read();     // the copies have read this CTA's pieces
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (RV_PAIR) mbar_arrive_cluster(pair_map(tempty0 + 8 * buf, 0));    // the first CTA's barrier counts both CTAs' warps
                else mbar_arrive(tempty0 + 8 * buf);
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tcgen05_fence_before();
    __syncthreads();
    // a pair leaves together: neither CTA frees tensor memory or exits while the other may still use its shared memory or barriers
    if (RV_PAIR) pair_sync();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::" CTA_GROUP ".sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
    if (threadIdx.x == 0 && abort_flag != 0 && p.status) atomicCAS(p.status, 0, abort_flag);
}

// ---------------------------------------------------------------- host side
// One CTA per tile and SM, or (RV_PAIR) one cluster of two CTAs per tile and pair of SMs.
static int launch_gemm(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmParams& p, int max_ctas, cudaStream_t stream) {
    const int smem = STAGES * STAGE_BYTES + 1024;
    // (the largest a launch may ask for: the pieces of an exchange between four CTAs)
    const int most_pieces = 2 * 3 * BM * (BN / 4 + 4) * 4 + 1024;
    static RvPerDevice configured;
    if (int e = rv_configure_smem(configured, gemm_tcgen05_kernel, most_pieces > smem ? most_pieces : smem)) return e;
    int workers = p.m_tiles * p.n_tiles;
#if !RV_PAIR
    if (p.splits > 1) {      // one cluster of `splits` CTAs per tile; the pieces of the exchange lie where the stages were
        const int pieces = 2 * (p.splits - 1) * BM * (BN / p.splits + 4) * 4 + 1024;
        const int split_smem = pieces > smem ? pieces : smem;
        RV_LAUNCH_ST = rv_launch_cluster(gemm_tcgen05_kernel, dim3(workers * p.splits), dim3(NUM_THREADS), split_smem, stream,
                                         (unsigned)p.splits, map_a, map_b, p);
        return rv_launch_status();
    }
#endif
    const int limit = (max_ctas > 0 ? max_ctas : rv_sm_count()) / (RV_PAIR ? 2 : 1);
    if (workers > limit) workers = limit;
    if (workers < 1) workers = 1;
#if RV_PAIR
    RV_LAUNCH_ST = rv_launch_cluster(gemm_tcgen05_kernel, dim3(2 * workers), dim3(NUM_THREADS), smem, stream, 2u, map_a, map_b, p);
#else
    RV_LAUNCH_ST = rv_launch(gemm_tcgen05_kernel, dim3(workers), dim3(NUM_THREADS), smem, stream, map_a, map_b, p);
#endif
    return rv_launch_status();
}

// 1 if this library was built for pairs of CTAs
RV_EXPORT int rv_gemm_tcgen05_is_pair() { return RV_PAIR; }

// epilogue: 0 plain, 1 + residual (bf16 [M, N]), 2 gated (W rows [gate | up], out has N/2 columns).
// status: optional device int that receives a non-zero code if a wait inside the kernel gave up.
// splits (both entry points): 1, or 2 / 4 on the build for single CTAs: the CTAs of a tile share its K as a cluster
// (see GemmParams); not with the gated epilogue, and with the rotary one only while a CTA's columns hold whole heads.
static int check_splits(int splits, int K, int epilogue, int hd) {
    if (splits == 1) return RV_OK;
    if (RV_PAIR || (splits != 2 && splits != 4) || epilogue == EPI_GATED) return RV_ERR_UNSUPPORTED;
    if ((K + BK - 1) / BK < splits) return RV_ERR_UNSUPPORTED;
    if (epilogue == EPI_ROPE && (BN / splits) % hd) return RV_ERR_UNSUPPORTED;
    return RV_OK;
}

RV_EXPORT int rv_gemm_tcgen05_bf16(const void* x, const void* w, const void* residual, void* out, int out_f32,
                                   int M, int N, int K, int epilogue, int* status, int max_ctas, int splits,
                                   cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0) return RV_ERR_BAD_SIZE;
    if (int e = check_splits(splits, K, epilogue, 0)) return e;
    if (K % 8) return RV_ERR_UNSUPPORTED;                          // rows must start on 16-byte boundaries
    if (epilogue == EPI_GATED && (N & 1)) return RV_ERR_BAD_SIZE;
    if (epilogue == EPI_RESIDUAL && (!residual || out_f32)) return RV_ERR_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out) |
         reinterpret_cast<uintptr_t>(residual)) % 16)
        return RV_ERR_ALIGNMENT;
    if (M == 0) return RV_OK;
    alignas(64) CUtensorMap map_a, map_b;
    int st = rv_make_bf16_map(&map_a, x, M, K, BM);
    if (st != RV_OK) return st;
    st = rv_make_bf16_map(&map_b, w, N, K, BN / 2);
    if (st != RV_OK) return st;
    GemmParams p = {};
    p.out = out; p.residual = epilogue == EPI_RESIDUAL ? (const __nv_bfloat16*)residual : nullptr;
    p.status = status; p.M = M; p.N = N; p.K = K; p.out_f32 = out_f32; p.epilogue = epilogue;
    p.splits = splits;
    p.m_tiles = (M + TILE_ROWS - 1) / TILE_ROWS;
    // gated: a tile is 128 gate rows and the 128 up rows of the same output columns; gate rows past
    // N/2 read up rows, whose products the epilogue never stores
    p.n_tiles = epilogue == EPI_GATED ? (N / 2 + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN;
    return launch_gemm(map_a, map_b, p, max_ctas, stream);
}

// The q/k/v product of an attention layer for many rows, with bias, rotation and the cache write in
// its epilogue.  w: [(nh + 2 nkv) * hd, K], hd 64, 128 or 256; q_out: [M, nh * hd]; kv_cache:
// [pages, 2, nkv, page_size, hd]; cos_t / sin_t: [table_rows, hd / 2] floats or both nullptr.
RV_EXPORT int rv_gemm_tcgen05_qkv_rope(const void* x, const void* w, const void* bias, int bias_dtype,
                                       const int* positions, const float* cos_t, const float* sin_t,
                                       const int* slot_mapping, void* kv_cache, void* q_out, int M, int K,
                                       int nh, int nkv, int hd, int page_size, int table_rows, int* status,
                                       int max_ctas, int splits, cudaStream_t stream) {
    if (M < 0 || K <= 0 || nh <= 0 || nkv <= 0 || page_size <= 0 || table_rows <= 0) return RV_ERR_BAD_SIZE;
    if (int e = check_splits(splits, K, EPI_ROPE, hd)) return e;
    if (hd != 64 && hd != 128 && hd != 256) return RV_ERR_UNSUPPORTED;     // a head's halves are whole 32-column chunks of one tile
    if (hd > BN) return RV_ERR_UNSUPPORTED;                                // (a narrow-tile build cannot hold a head of 256)
    if (K % 8) return RV_ERR_UNSUPPORTED;
    if ((cos_t == nullptr) != (sin_t == nullptr)) return RV_ERR_BAD_SIZE;
    if (!positions || !slot_mapping || !kv_cache || !q_out) return RV_ERR_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(q_out) |
         reinterpret_cast<uintptr_t>(kv_cache) | reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t)) % 16)
        return RV_ERR_ALIGNMENT;
    if (M == 0) return RV_OK;
    const int N = (nh + 2 * nkv) * hd;
    alignas(64) CUtensorMap map_a, map_b;
    int st = rv_make_bf16_map(&map_a, x, M, K, BM);
    if (st != RV_OK) return st;
    st = rv_make_bf16_map(&map_b, w, N, K, BN / 2);
    if (st != RV_OK) return st;
    GemmParams p = {};
    p.status = status; p.M = M; p.N = N; p.K = K; p.epilogue = EPI_ROPE;
    p.splits = splits;
    p.m_tiles = (M + TILE_ROWS - 1) / TILE_ROWS;
    p.n_tiles = (N + BN - 1) / BN;
    p.bias = bias; p.bias_dtype = bias_dtype;
    p.q_out = (__nv_bfloat16*)q_out; p.kv_cache = (__nv_bfloat16*)kv_cache;
    p.positions = positions; p.slot_mapping = slot_mapping; p.cos_t = cos_t; p.sin_t = sin_t;
    p.nh = nh; p.nkv = nkv; p.hd = hd; p.page_size = page_size; p.table_rows = table_rows;
    return launch_gemm(map_a, map_b, p, max_ctas, stream);
}
