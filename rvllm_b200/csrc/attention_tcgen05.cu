// Paged flash attention for prompt portions on the fifth-generation tensor cores (bfloat16).
//
// A CTA owns up to 128 rows - (token, query head) pairs of ONE key/value head, the G = nh / nkv heads
// of a group packed side by side: floor(128 / G) whole tokens, so 128 rows where G divides 128 and for
// instance 126 (18 tokens) for G = 7; the rows left over are zeros that nothing reads back - and walks
// the sequence's keys in tiles of 64:
//   S = Q K^T        tcgen05.mma, Q [128 x hd] and K [64 x hd] K-major in shared memory (TMA,
//                    128-byte swizzle), S [128 x 64] float in tensor memory;
//   softmax          four warps, one thread per row: tcgen05.ld of the row, scale, causal / window
//                    mask, running maximum and sum in float, P = exp2(s - m) packed as bfloat16
//                    pairs and written back into tensor memory (tcgen05.st) over the first half of
//                    the S buffer it came from;
//   O += P V         tcgen05.mma with P as the A operand FROM TENSOR MEMORY and V [64 keys x hd] as
//                    the MN-major B operand straight from the cache's [key][hd] pages, O [128 x hd]
//                    float accumulated in tensor memory.
// P never passes through shared memory, and because P(i) lives in S buffer i mod 2, the softmax of
// tile i + 1 does not have to wait for the P V product of tile i: softmax and tensor core run side
// by side.  The reference maximum of a row is only raised when the true maximum has grown by more
// than 2^8 (then O is rescaled in tensor memory), so most tiles need no pass over O; the final
// division by the row sum uses the same reference.
//
// Eight warps, every one a chain of waits and a little work per tile, so that none of them is
// slower than the softmax: four softmax warps (one warpgroup); a loader of Q and the keys and a
// loader of the values (one TMA box per (page, half of hd) through the block table, whose entries
// are read a tile ahead; rings of NK and NV stages); a warp whose one thread issues S = Q K^T and
// one that issues O += P V (S(i) overwrites P(i - 2), so the first follows the second's o_full
// barrier).  The second warpgroup hands most of its registers to the softmax warps (setmaxnreg).
// Two CTAs fit an SM, so the softmax of one overlaps that of the other.  Every mbarrier wait is
// bounded.
//
// Rule as in attention_flash.cu (v3/kernels/paged_attention_sm89.cu:277-308 of the reference):
// token i of the step's q_len tokens sits at p = ctx_len - q_len + i and sees keys (p - window, p].
// Cache layer layout: [num_pages, 2 (k, v), nkv, page_size, HEAD_DIM].
#include "common.cuh"
#include "tcgen05.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "this kernel is built for head sizes 64 and 128");

#define ROWS 128
#define KV_TILE 64
#define SOFTMAX_WARPS 4
#define LOADER_WARP SOFTMAX_WARPS               // Q and the keys (and the tensor memory's allocation)
#define VLOADER_WARP (SOFTMAX_WARPS + 1)       // the values
#define QK_WARP (SOFTMAX_WARPS + 2)            // issues S = Q K^T
#define PV_WARP (SOFTMAX_WARPS + 3)            // issues O += P V
#define HALVES (HEAD_DIM / 64)                 // 64-element (128-byte) slabs of the head dimension
#define Q_BYTES (ROWS * HEAD_DIM * 2)
#define KV_BYTES (KV_TILE * HEAD_DIM * 2)      // one of K or V for a tile
#define NUM_THREADS (32 * (SOFTMAX_WARPS + 4)) // two warpgroups: the softmax warps; 2 loader warps and 2 MMA warps
// Two CTAs fit an SM, so a thread starts with 128 registers; the four warps that load and issue give
// most of theirs back and the softmax warps take them (setmaxnreg works on whole warpgroups).
#define REGS_SOFTMAX 200
#define REGS_OTHERS 56
#define TMEM_COLS 256
#define S_COL 0                   // two S buffers of 64 columns; P (bf16 pairs) reuses the first 32 columns of each
#define O_COL 128
// Stages of the key ring and of the value ring: what fits beside Q with two CTAs on an SM.
#define NK (HEAD_DIM == 128 ? 3 : 4)
#define NV (HEAD_DIM == 128 ? 2 : 4)
// mbarriers, by their index
#define B_Q 0
#define B_K 1                      // keys of a stage have landed [NK]
#define B_KFREE (B_K + NK)         // the S product that read a stage has finished [NK]
#define B_V (B_KFREE + NK)         // values of a stage have landed [NV]
#define B_VFREE (B_V + NV)         // the P V product that read a stage has finished [NV]
#define B_SFULL (B_VFREE + NV)     // [2] each from here on
#define B_OFULL (B_SFULL + 2)
#define B_PFULL (B_OFULL + 2)
#define NUM_BARS (B_PFULL + 2)
static_assert(NUM_BARS <= 30, "the barriers, the tensor-memory address and the abort flag share 256 bytes");
#define RESCALE_LOG2 8.0f

struct AttnParams {
    const int* block_tables;
    const int* cu_seqlens;
    const int* ctx_lens;
    __nv_bfloat16* out;
    int* status;
    int nh, nkv, page_shift, page_size, max_blocks;
    float scale_log2e;
    int window;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
// 2^x by the special-function unit; -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// the largest of three in one instruction
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// two multiply-adds, two additions in one instruction each (packed pairs of floats)
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b, float c) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}" : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1) {
    asm("{\n\t.reg .b64 ra, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\tadd.rn.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "+f"(d0), "+f"(d1) : "f"(a0), "f"(a1));
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows in the 128 lanes, 16 bf16 of K in 8 columns) from tensor memory
__device__ __forceinline__ void tcgen05_mma_bf16_ts(uint32_t tmem_c, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                                    uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_c), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// MN-major operand with 128-byte swizzle (V as [key][hd]): 64 consecutive hd elements are one
// 128-byte row; groups of 8 keys are 1024 bytes apart (stride offset); the next 64 hd elements
// start `lbo_bytes` further (leading offset).
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__global__ void __launch_bounds__(NUM_THREADS, 2)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                         const AttnParams p) {
    // All shared memory is dynamic (no static arrays), so that the tiles start on the 1024-byte
    // boundary the 128-byte swizzle needs without a pad, and two CTAs fit an SM.
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* q_s = smem_raw;                           // [HALVES][128 rows x 128 B]
    unsigned char* k_s = q_s + Q_BYTES;                      // [NK stages][HALVES][KV_TILE keys x 128 B]
    unsigned char* v_s = k_s + NK * KV_BYTES;                // [NV stages][HALVES][KV_TILE keys x 128 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + NV * KV_BYTES);
    uint32_t& tmem_base_slot = *reinterpret_cast<uint32_t*>(bars + 30);
    volatile int& abort_flag = *reinterpret_cast<volatile int*>(bars + 31);

    rv_pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { tma_prefetch_descriptor(&map_q); tma_prefetch_descriptor(&map_kv); }
    const uint32_t bar_q = smem_u32(&bars[B_Q]), bar_k0 = smem_u32(&bars[B_K]);
    const uint32_t bar_kfree0 = smem_u32(&bars[B_KFREE]), bar_v0 = smem_u32(&bars[B_V]);
    const uint32_t bar_vfree0 = smem_u32(&bars[B_VFREE]);
    const uint32_t bar_s_full0 = smem_u32(&bars[B_SFULL]);
    // The P V product of tile i reports on o_full[i mod 2], P of tile i on p_full[i mod 2]: two barriers each,
    // because a waiter may be a tile behind the one that arrives (with one barrier it could not tell phase
    // i - 1 from phase i + 1; a softmax warp may also run one tile ahead of the slowest, and its arrival for
    // tile i + 1 must not be counted among the four of tile i).
    const uint32_t bar_o_full0 = smem_u32(&bars[B_OFULL]), bar_p_full0 = smem_u32(&bars[B_PFULL]);

    // Row tiles late in the prompt see the most keys.  CTAs are handed out in the order of their
    // linear index (x fastest), so the row tile is the slowest index, counted down: all heads' and
    // sequences' heaviest tiles start first and the light ones fill the end (with the row tile
    // as the fastest index the last heads' heavy tiles started late and set the kernel's length).
    const int kvh = blockIdx.x, seq = blockIdx.y, tile_m = gridDim.z - 1 - blockIdx.z;
    const int G = p.nh / p.nkv;
    rv_pdl_wait();
    const int ctx = p.ctx_lens[seq];
    const int q_start = p.cu_seqlens[seq];
    const int q_len = p.cu_seqlens[seq + 1] - q_start;
    const int rows_total = q_len * G;
    const int tile_rows = (ROWS / G) * G;                               // whole tokens only
    const int row0 = tile_m * tile_rows;
    if (q_len <= 1 || ctx <= 0 || row0 >= rows_total) return;          // one-token sequences go to the decode kernel

    const int last_row = min(rows_total, row0 + tile_rows) - 1;
    const int pos_first = ctx - q_len + row0 / G, pos_last = ctx - q_len + last_row / G;
    const int key_lo = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    const int key_hi = pos_last + 1;
    const int t_begin = key_lo / KV_TILE, t_end = (key_hi + KV_TILE - 1) / KV_TILE;
    const int* table = p.block_tables + (size_t)seq * p.max_blocks;

    if (tid == 0) {
        abort_flag = 0;
        mbar_init(bar_q, 1);
        for (int i = 0; i < NK; ++i) { mbar_init(bar_k0 + 8 * i, 1); mbar_init(bar_kfree0 + 8 * i, 1); }
        for (int i = 0; i < NV; ++i) { mbar_init(bar_v0 + 8 * i, 1); mbar_init(bar_vfree0 + 8 * i, 1); }
        mbar_init(bar_s_full0, 1); mbar_init(bar_s_full0 + 8, 1);
        // the softmax warps arrive once per warp (after a warp barrier), not once per thread
        mbar_init(bar_p_full0, SOFTMAX_WARPS); mbar_init(bar_p_full0 + 8, SOFTMAX_WARPS);
        mbar_init(bar_o_full0, 1); mbar_init(bar_o_full0 + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == LOADER_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    // value tiles start as zeros: a page that is not loaded (beyond the context, or given back by
    // a window) must not meet a probability of zero with a NaN
    for (int i = tid; i < NV * KV_BYTES / 16; i += NUM_THREADS) reinterpret_cast<uint4*>(v_s)[i] = make_uint4(0, 0, 0, 0);
    // ... and so do the query rows that the box of whole tokens leaves over (a row is 128 bytes in
    // each half of the head, whatever the swizzle does inside it)
    for (int i = tid; i < (ROWS - tile_rows) * 8 * HALVES; i += NUM_THREADS) {
        const int h = i / ((ROWS - tile_rows) * 8), j = i - h * ((ROWS - tile_rows) * 8);
        reinterpret_cast<uint4*>(q_s + h * (ROWS * 128) + tile_rows * 128)[j] = make_uint4(0, 0, 0, 0);
    }
    fence_async_smem();
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const int box_keys = p.page_size < KV_TILE ? p.page_size : KV_TILE;     // keys one TMA box brings
    const int boxes = KV_TILE / box_keys;

    const int n_it = t_end - t_begin;
#ifdef ATTN_TRACE
    const int tr0 = p.status ? p.status[1] : 0, tr_z = p.status ? p.status[2] : 0;
    if (p.status && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && (int)blockIdx.z == tr_z) { p.status[4] = (int)clock64(); p.status[6] = n_it; unsigned long long g; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g)); p.status[3] = (int)(unsigned)g; }
#endif
    int tiles_issued = 0;             // by this warp, if it is a loader
    if (warp == LOADER_WARP || warp == VLOADER_WARP) {
        // ------------------------------------------------------------ loader warps: TMA, one for keys, one for values
        // Lane 0 waits on barriers (the result is broadcast); the lanes share the TMA boxes of a tile,
        // one (page, both halves of hd) each.  The tile that follows a stage's tile (NK or NV tiles on)
        // is loaded when the product that read the stage has finished; each stage reports on a barrier
        // of its own, so that a product can never be two phases ahead of its loader.  The block-table
        // entries of a load are read a turn before it is issued: a loader is one chain of waits and
        // loads, and has to stay ahead of the products.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_OTHERS));
        const int which = warp == LOADER_WARP ? 0 : 1;
        const int stages = which == 0 ? NK : NV;
        const uint32_t bar_full0 = which == 0 ? bar_k0 : bar_v0, bar_free0 = which == 0 ? bar_kfree0 : bar_vfree0;
        const uint32_t ring = smem_u32(which == 0 ? k_s : v_s);
        auto wait_all = [&](uint32_t bar, uint32_t parity, int code) -> bool {
            int ok_l = 1;
            if (lane == 0) ok_l = mbar_wait(bar, parity, &abort_flag, code) ? 1 : 0;
            return __shfl_sync(0xffffffffu, ok_l, 0) != 0;
        };
        auto lookup = [&](int t) -> int {               // this lane's page of tile t, or -1
            const int key = t * KV_TILE + lane * box_keys;
            return (lane < boxes && key < key_hi && key + box_keys > key_lo) ? __ldg(table + (key >> p.page_shift)) : -1;
        };
        auto issue = [&](int t, int stage, int page) {
            const uint32_t bar = bar_full0 + 8 * stage;
            const uint32_t dst0 = ring + (uint32_t)stage * KV_BYTES;
            const int key = t * KV_TILE + lane * box_keys;
            const unsigned mask = __ballot_sync(0xffffffffu, page >= 0);
            if (lane == 0) mbar_expect_tx(bar, (uint32_t)__popc(mask) * HALVES * (uint32_t)box_keys * 128u);
            __syncwarp();
            if (page >= 0) {
                const int row = ((page * 2 + which) * p.nkv + kvh) * p.page_size + (key & (p.page_size - 1));
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
                    tma_load_2d(dst0 + (uint32_t)h * (KV_TILE * 128) + (uint32_t)lane * box_keys * 128, &map_kv, h * 64, row, bar);
            }
            __syncwarp();
        };
        // Q: one box of [64 hd, G heads, floor(128 / G) tokens] per half of the head dimension
        if (which == 0 && lane == 0) {
            mbar_expect_tx(bar_q, (uint32_t)tile_rows * HEAD_DIM * 2);
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
                tma_load_3d(smem_u32(q_s) + h * (ROWS * 128), &map_q, h * 64, kvh * G, q_start + row0 / G, bar_q);
        }
        for (int i = 0; i < stages && i < n_it; ++i, ++tiles_issued) issue(t_begin + i, i, lookup(t_begin + i));
        int page = stages < n_it ? lookup(t_begin + stages) : -1;
        int stage = 0;
        uint32_t phase = 0;
        for (int e = 0; e + stages < n_it; ++e) {
            const int next = e + 1 + stages < n_it ? lookup(t_begin + e + 1 + stages) : -1;
#ifdef ATTN_TRACE
            const bool trl = p.status && blockIdx.x == 0 && blockIdx.y == 0 && (int)blockIdx.z == tr_z && e >= tr0 && e < tr0 + 24 && lane == 0;
            if (trl) p.status[8 + 800 + 800 * which + (e - tr0) * 5 + 0] = (int)clock64();
#endif
            if (!wait_all(bar_free0 + 8 * stage, phase, 3 + which)) break;
#ifdef ATTN_TRACE
            if (trl) p.status[8 + 800 + 800 * which + (e - tr0) * 5 + 1] = (int)clock64();
#endif
            issue(t_begin + e + stages, stage, page);
            ++tiles_issued;
#ifdef ATTN_TRACE
            if (trl) p.status[8 + 800 + 800 * which + (e - tr0) * 5 + 2] = (int)clock64();
#endif
            page = next;
            if (++stage == stages) { stage = 0; phase ^= 1; }
        }
    } else if (warp == QK_WARP) {
        // ------------------------------------------------------------ first MMA warp: S = Q K^T, one thread issues
        // S(i) goes into buffer i mod 2, over P(i - 2): the product that read P(i - 2) must have finished
        // (o_full, which this thread follows phase by phase).  The two kinds of product have a warp each
        // because a thread that waits on four barriers and issues twelve products a tile is, by itself,
        // slower than the softmax warps.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_OTHERS));
        if (lane == 0) {
            const uint32_t idesc_s = umma_idesc_bf16(ROWS, KV_TILE);
            bool ok = mbar_wait(bar_q, 0, &abort_flag, 1);
            int k_stage = 0;
            uint32_t k_phase = 0;
            for (int i = 0; i < n_it && ok; ++i) {
                const int buf = i & 1;
#ifdef ATTN_TRACE
                const bool trm = p.status && blockIdx.x == 0 && blockIdx.y == 0 && (int)blockIdx.z == tr_z && i >= tr0 && i < tr0 + 24;
                if (trm) p.status[8 + 400 + (i - tr0) * 5 + 0] = (int)clock64();
#endif
                if (!(ok = mbar_wait(bar_k0 + 8 * k_stage, k_phase, &abort_flag, 5))) break;
#ifdef ATTN_TRACE
                if (trm) p.status[8 + 400 + (i - tr0) * 5 + 1] = (int)clock64();
#endif
                if (i >= 2 && !(ok = mbar_wait(bar_o_full0 + 8 * buf, ((i - 2) >> 1) & 1, &abort_flag, 6))) break;
                tcgen05_fence_after();
#ifdef ATTN_TRACE
                if (trm) p.status[8 + 400 + (i - tr0) * 5 + 2] = (int)clock64();
#endif
#pragma unroll
                for (int h = 0; h < HALVES; ++h) {
                    const uint64_t dq = umma_desc(smem_u32(q_s) + h * (ROWS * 128));
                    const uint64_t dk = umma_desc(smem_u32(k_s) + k_stage * KV_BYTES + h * (KV_TILE * 128));
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        tcgen05_mma_bf16(tmem_base + S_COL + buf * KV_TILE, dq + (uint64_t)(2 * j), dk + (uint64_t)(2 * j),
                                         idesc_s, (h | j) != 0);
                }
                tcgen05_commit(bar_s_full0 + 8 * buf);
                tcgen05_commit(bar_kfree0 + 8 * k_stage);
#ifdef ATTN_TRACE
                if (trm) p.status[8 + 400 + (i - tr0) * 5 + 3] = (int)clock64();
#endif
                if (++k_stage == NK) { k_stage = 0; k_phase ^= 1; }
            }
        }
    } else if (warp == PV_WARP) {
        // ------------------------------------------------------------ second MMA warp: O += P V
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_OTHERS));
        if (lane == 0) {
            const uint32_t idesc_o = umma_idesc_bf16(ROWS, HEAD_DIM) | (1u << 16);       // B is MN-major
            bool ok = true;
            int v_stage = 0;
            uint32_t v_phase = 0;
            for (int it = 0; it < n_it && ok; ++it) {
                const int b = it & 1;
#ifdef ATTN_TRACE
                const bool trm = p.status && blockIdx.x == 0 && blockIdx.y == 0 && (int)blockIdx.z == tr_z && it >= tr0 && it < tr0 + 24;
                if (trm) p.status[8 + 2400 + (it - tr0) * 5 + 0] = (int)clock64();
#endif
                if (!(ok = mbar_wait(bar_v0 + 8 * v_stage, v_phase, &abort_flag, 7))) break;
#ifdef ATTN_TRACE
                if (trm) p.status[8 + 2400 + (it - tr0) * 5 + 1] = (int)clock64();
#endif
                // once the softmax warps have written P (and rescaled O if they had to)
                if (!(ok = mbar_wait(bar_p_full0 + 8 * b, (it >> 1) & 1, &abort_flag, 8))) break;
                tcgen05_fence_after();
#ifdef ATTN_TRACE
                if (trm) p.status[8 + 2400 + (it - tr0) * 5 + 2] = (int)clock64();
#endif
                const uint32_t tp = tmem_base + S_COL + b * KV_TILE;     // P(it): bf16 pairs in the first half of S buffer b
                const uint64_t dv = umma_desc_mn(smem_u32(v_s) + v_stage * KV_BYTES, KV_TILE * 128);
#pragma unroll
                for (int j = 0; j < KV_TILE / 16; ++j)   // 16 keys per MMA: 8 columns along P's rows, 2048 bytes down V
                    tcgen05_mma_bf16_ts(tmem_base + O_COL, tp + 8 * j, dv + (uint64_t)(128 * j), idesc_o, (it | j) != 0);
                tcgen05_commit(bar_vfree0 + 8 * v_stage);
                tcgen05_commit(bar_o_full0 + 8 * b);
#ifdef ATTN_TRACE
                if (trm) p.status[8 + 2400 + (it - tr0) * 5 + 3] = (int)clock64();
#endif
                if (++v_stage == NV) { v_stage = 0; v_phase ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------ softmax warps: one thread per row
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_SOFTMAX));
        const int row_l = warp * 32 + lane;                  // row of the tile = TMEM lane
        const int r = row0 + row_l;                          // packed row
        const bool in_range = row_l < tile_rows && r < rows_total;
        const int tok_i = in_range ? r / G : 0;
        const int head = kvh * G + (in_range ? r - tok_i * G : 0);
        const int pos = in_range ? ctx - q_len + tok_i : -1;
        const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
        const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
        float m_ref = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int t = t_begin; t < t_end; ++t) {
            const int it = t - t_begin;
            const int sb = it & 1;
#ifdef ATTN_TRACE
            const bool tr = p.status && blockIdx.x == 0 && blockIdx.y == 0 && (int)blockIdx.z == tr_z && tid == 0 && it >= tr0 && it < tr0 + 24;
            if (tr) p.status[8 + (it - tr0) * 5 + 0] = (int)clock64();
#endif
            if (!mbar_wait(bar_s_full0 + 8 * sb, (it >> 1) & 1, &abort_flag, 9)) { ok = false; break; }
#ifdef ATTN_TRACE
            if (tr) p.status[8 + (it - tr0) * 5 + 1] = (int)clock64();
#endif
            tcgen05_fence_after();
            uint32_t s0[32], s1[32];
            tmem_ld_32x32(t_lane + S_COL + sb * KV_TILE, s0);
            tmem_ld_32x32(t_lane + S_COL + sb * KV_TILE + 32, s1);
            tmem_ld_wait();
            tcgen05_fence_before();
            __syncwarp();
            const int key0 = t * KV_TILE;
            // Scores stay raw in the registers; scale and reference maximum are applied in one FMA
            // before the exponential.  Only tiles that cross the row's visible range need masks.
            if (!(key0 + KV_TILE - 1 <= pos && key0 >= lo)) {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int ka = key0 + e, kb = key0 + 32 + e;
                    if (!(ka <= pos && ka >= lo)) s0[e] = 0xff800000u;        // -inf
                    if (!(kb <= pos && kb >= lo)) s1[e] = 0xff800000u;
                }
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};     // four chains: one would be a chain of latencies
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
                mx[0] = max3(mx[0], __uint_as_float(s0[e]), __uint_as_float(s0[e + 1]));
                mx[1] = max3(mx[1], __uint_as_float(s0[e + 2]), __uint_as_float(s0[e + 3]));
                mx[2] = max3(mx[2], __uint_as_float(s1[e]), __uint_as_float(s1[e + 1]));
                mx[3] = max3(mx[3], __uint_as_float(s1[e + 2]), __uint_as_float(s1[e + 3]));
            }
            const float m_raw = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            const float m_tile = m_raw * p.scale_log2e;       // the scale is positive: the maximum commutes
            // raise the reference maximum only when it is far behind: O then needs a pass
            const bool first_data = m_ref == -INFINITY && m_tile > -INFINITY;
            const bool raise = first_data || m_tile > m_ref + RESCALE_LOG2;
            float factor = 1.f;
            if (raise) {
                factor = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - m_tile);
                m_ref = m_tile;
                l_run *= factor;
            }
            // P(it) goes into S buffer sb, which no product reads any more (P(it - 2) was consumed before
            // S(it) was produced), so only a rescale of O has to wait for the P V product of the tile before.
#ifdef ATTN_TRACE
            if (tr) p.status[8 + (it - tr0) * 5 + 2] = (int)clock64();
#endif
            const bool any_raise = __any_sync(0xffffffffu, raise && it > 0);
            if (any_raise) {
                // O is rescaled: the product of the tile before must have finished.  The one before that
                // has (S(it - 1) was only issued after it), and the one after cannot have started (it needs
                // this warp's P), so the parity of o_full[(it - 1) mod 2] cannot be mistaken.
                if (!mbar_wait(bar_o_full0 + 8 * ((it - 1) & 1), ((it - 1) >> 1) & 1, &abort_flag, 11)) { ok = false; break; }
                tcgen05_fence_after();
#pragma unroll
                for (int c = 0; c < HEAD_DIM; c += 32) {
                    uint32_t o[32];
                    tmem_ld_32x32(t_lane + O_COL + c, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * factor);
                    tmem_st_32x32(t_lane + O_COL + c, o);
                }
                tmem_st_wait();
                tcgen05_fence_before();
            }
#ifdef ATTN_TRACE
            if (tr) p.status[8 + (it - tr0) * 5 + 3] = (int)clock64();
#endif
            const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
            float l_tile = 0.f, l_tile2 = 0.f;
            uint32_t pk[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {                   // keys 2j and 2j + 1 of the tile: one column of P
                const int e = 2 * j;
                float a0, a1;
                fma2(a0, a1, __uint_as_float(e < 32 ? s0[e] : s1[e - 32]), __uint_as_float(e + 1 < 32 ? s0[e + 1] : s1[e + 1 - 32]),
                     p.scale_log2e, neg_m);
                const float x0 = fast_exp2(a0), x1 = fast_exp2(a1);
                add2(l_tile, l_tile2, x0, x1);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(x0, x1);
                pk[j] = *reinterpret_cast<uint32_t*>(&h2);
            }
            l_tile += l_tile2;
            l_run += l_tile;
            tmem_st_32x32(t_lane + S_COL + sb * KV_TILE, pk);
            tmem_st_wait();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_full0 + 8 * sb);
#ifdef ATTN_TRACE
            if (tr) p.status[8 + (it - tr0) * 5 + 4] = (int)clock64();
#endif
        }
        if (ok) {
            // the last product (the one before it, on the other barrier, finished earlier: products run in order)
            ok = mbar_wait(bar_o_full0 + 8 * ((n_it - 1) & 1), ((n_it - 1) >> 1) & 1, &abort_flag, 10);
            tcgen05_fence_after();
            if (ok) {
                const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
                __nv_bfloat16* dst = p.out + ((size_t)(q_start + tok_i) * p.nh + head) * HEAD_DIM;
#pragma unroll
                for (int c = 0; c < HEAD_DIM; c += 32) {
                    uint32_t o[32];
                    tmem_ld_32x32(t_lane + O_COL + c, o);
                    tmem_ld_wait();
                    if (in_range) {
#pragma unroll
                        for (int v4 = 0; v4 < 4; ++v4) {
                            uint4 v;
                            uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(o[v4 * 8 + 2 * j]) * inv,
                                                                          __uint_as_float(o[v4 * 8 + 2 * j + 1]) * inv);
                                w[j] = *reinterpret_cast<uint32_t*>(&h2);
                            }
                            *reinterpret_cast<uint4*>(dst + c + v4 * 8) = v;
                        }
                    }
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (abort_flag != 0) {
        // A wait gave up somewhere: tiles may still be on their way into this CTA's shared memory with nobody
        // left to wait for them.  Their loaders do (bounded, without touching the flag) before the CTA ends.
        if ((warp == LOADER_WARP || warp == VLOADER_WARP) && lane == 0) {
            volatile int ignore = 0;
            const int stages = warp == LOADER_WARP ? NK : NV;
            const uint32_t full0 = warp == LOADER_WARP ? bar_k0 : bar_v0;
            if (warp == LOADER_WARP) mbar_wait(bar_q, 0, &ignore, 0);
            for (int i = max(0, tiles_issued - stages); i < tiles_issued; ++i)
                mbar_wait(full0 + 8 * (i % stages), (i / stages) & 1, &ignore, 0);
        }
        __syncthreads();
    }
#ifdef ATTN_TRACE
    if (p.status && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && (int)blockIdx.z == tr_z) { p.status[5] = (int)clock64(); unsigned long long g; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g)); p.status[7] = (int)(unsigned)g; }
#endif
    if (warp == LOADER_WARP) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
    if (tid == 0 && abort_flag != 0 && p.status) atomicCAS(p.status, 0, abort_flag);
}

// ---------------------------------------------------------------- host side
static int make_q_map(CUtensorMap* map, const void* q, int n_tokens, int nh, int G) {
    RvEncodeTiledFn fn = rv_encode_fn();
    if (!fn) return RV_ERR_UNSUPPORTED;
    const cuuint64_t dims[3] = {HEAD_DIM, (cuuint64_t)nh, (cuuint64_t)n_tokens};
    const cuuint64_t strides[2] = {HEAD_DIM * 2, (cuuint64_t)nh * HEAD_DIM * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(ROWS / G)};
    const cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? RV_OK : RV_ERR_BAD_SIZE;
}

RV_EXPORT int rv_attention_tcgen05_head_dim() { return HEAD_DIM; }

// Attention of the sequences that bring more than one token to the step (the others are left to
// the decode kernel).  Refuses (RV_ERR_UNSUPPORTED) what it is not built for: a head size other
// than HEAD_DIM, a group of more than 128 heads, pages of fewer than 8 keys.
RV_EXPORT int rv_attention_tcgen05(const void* q, const void* cache, long long num_pages, const int* block_tables,
                                   const int* cu_seqlens, const int* ctx_lens, void* out, int n_tokens, int num_seqs,
                                   int nh, int nkv, int hd, int page_size, int max_blocks, float scale, int window,
                                   int max_q_len, int* status, cudaStream_t stream) {
    if (hd != HEAD_DIM) return RV_ERR_UNSUPPORTED;
    if (n_tokens < 0 || num_seqs < 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || max_blocks <= 0 || max_q_len <= 0)
        return RV_ERR_BAD_SIZE;
    const int G = nh / nkv;
    if (G > ROWS) return RV_ERR_UNSUPPORTED;
    if ((page_size & (page_size - 1)) || page_size < 8) return RV_ERR_UNSUPPORTED;
    if (num_seqs > 65535 || nkv > 65535) return RV_ERR_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(out)) % 16)
        return RV_ERR_ALIGNMENT;
    if (n_tokens == 0 || num_seqs == 0) return RV_OK;
    alignas(64) CUtensorMap map_q, map_kv;
    int st = make_q_map(&map_q, q, n_tokens, nh, G);
    if (st != RV_OK) return st;
    st = rv_make_bf16_map(&map_kv, cache, num_pages * 2 * nkv * page_size, HEAD_DIM, page_size < KV_TILE ? page_size : KV_TILE);
    if (st != RV_OK) return st;
    AttnParams p;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.ctx_lens = ctx_lens; p.out = (__nv_bfloat16*)out;
    p.status = status; p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.max_blocks = max_blocks;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.window = window;
    const int smem = Q_BYTES + (NK + NV) * KV_BYTES + 256;
    static RvPerDevice configured;
    if (int e = rv_configure_smem(configured, attention_tcgen05_kernel, smem)) return e;
    const int tile_tokens = ROWS / G;
    const dim3 grid(nkv, num_seqs, (max_q_len + tile_tokens - 1) / tile_tokens);
    if (grid.y > 65535 || grid.z > 65535) return RV_ERR_UNSUPPORTED;
    RV_LAUNCH_ST = rv_launch(attention_tcgen05_kernel, grid, dim3(NUM_THREADS), smem, stream, map_q, map_kv, p);
    return rv_launch_status();
}
