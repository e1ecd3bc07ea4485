// Sampling over float logits [R, V]: greedy (lowest index wins ties, NaN never wins) and
// seeded temperature sampling with optional top-k / top-p, one block per row.
//
// Parameters per row as the reference's SamplingParams {temperature, top_k, top_p, seed}
// (v3/crates/rvllm-sampling/src/params.rs:7-28): temperature 0 means greedy.  The reference
// ships only an argmax kernel (kernels/argmax.cu:66-117; tie rule of its oracle,
// v3/crates/rvllm-fused/src/reference.rs:131-146); the rest is defined here:
//   p = softmax(logits / T) in float with the maximum subtracted;
//   top-k keeps the tokens at least as likely as the k-th most likely one;
//   top-p keeps the most likely tokens up to the first whose cumulated mass reaches top_p
//   (tokens exactly as likely as the last kept one stay in);
//   the draw is the first token, in vocabulary order, whose cumulated kept mass exceeds
//   u * (kept mass), with u = Philox4x32-10(key = seed, counter = index of the output token).
// The uniform depends on (seed, output index) only, never on the batch a row is sampled in.
//
// Rows with a top-k take two passes over the row (maximum + counts per bin of the top 12 bits of the
// ordered bit pattern, then the candidates from the k-th token's bin upwards and the whole mass), rows
// with a top-p alone three (arg-max, counts and fixed-point masses per bin, candidates); the at most
// 2,048 candidates are sorted and cut exactly in the first CTA's shared memory.  Rows whose candidates
// do not fit (a flat distribution under top-p alone, a k beyond 2,048) take the general search: eight
// passes of four bits over the row.  All sums that decide anything are integers or are added in a fixed
// order, so a token depends neither on the run nor on how many CTAs share the row.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Block-wide (value, index) arg-max: larger value wins, then lower index.
__device__ __forceinline__ void argmax_combine(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

__device__ int block_argmax(const float* row, int V, float* s_val, int* s_idx) {
    float best = -INFINITY;
    int idx = 0x7fffffff;
    if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        // 16-byte loads, two independent chains; indices rise within a chain, so a strict
        // comparison keeps the lowest index of equal values
        float b1 = -INFINITY;
        int i1 = 0x7fffffff;
        const float4* r4 = reinterpret_cast<const float4*>(row);
        const int n4 = V >> 2;
        int i = threadIdx.x;
        for (; i + (int)blockDim.x < n4; i += 2 * blockDim.x) {
            const float4 a = r4[i], b = r4[i + blockDim.x];
            const int ia = i * 4, ib = (i + blockDim.x) * 4;
            if (a.x > best) { best = a.x; idx = ia; }
            if (a.y > best) { best = a.y; idx = ia + 1; }
            if (a.z > best) { best = a.z; idx = ia + 2; }
            if (a.w > best) { best = a.w; idx = ia + 3; }
            if (b.x > b1) { b1 = b.x; i1 = ib; }
            if (b.y > b1) { b1 = b.y; i1 = ib + 1; }
            if (b.z > b1) { b1 = b.z; i1 = ib + 2; }
            if (b.w > b1) { b1 = b.w; i1 = ib + 3; }
        }
        if (i < n4) {
            const float4 a = r4[i];
            const int ia = i * 4;
            if (a.x > best || (a.x == best && ia < idx)) { best = a.x; idx = ia; }
            if (a.y > best || (a.y == best && ia + 1 < idx)) { best = a.y; idx = ia + 1; }
            if (a.z > best || (a.z == best && ia + 2 < idx)) { best = a.z; idx = ia + 2; }
            if (a.w > best || (a.w == best && ia + 3 < idx)) { best = a.w; idx = ia + 3; }
        }
        argmax_combine(best, idx, b1, i1);
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            if (v > best || (v == best && i < idx)) { best = v; idx = i; }   // NaN compares false
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_combine(best, idx, ov, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        best = lane < nw ? s_val[lane] : -INFINITY;
        idx = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            argmax_combine(best, idx, ov, oi);
        }
        if (lane == 0) { s_val[0] = best; s_idx[0] = idx == 0x7fffffff ? 0 : idx; }
    }
    __syncthreads();
    return s_idx[0];
}

// ---------------------------------------------------------------------------------------------
// One to eight CTAs per row.  A row is always cut into SAMPLE_SLICES contiguous slices of the
// vocabulary; every reduction over the row (arg-max, mass, the 16 + 16 sums of a pass of the
// threshold search, the kept mass) is done slice by slice by one block of SAMPLE_THREADS threads and
// the slices' results are combined in slice order.  With several CTAs per row (a thread-block
// cluster; each CTA owns SAMPLE_SLICES / CTAs neighbouring slices) each CTA writes its slices'
// results into every CTA's shared memory (st.shared::cluster), and one cluster barrier later all CTAs
// combine the same numbers in the same order and take the same decision.  So the sampled token does
// not depend on how many CTAs share the row, which the host chooses by the number of rows: one block
// per row is bound by its own instruction rate (125 tokens per thread and pass at a vocabulary of
// 128,256), eight CTAs make a pass eight times shorter.  The exchange buffers alternate between two
// copies, so that a CTA that is one step ahead never overwrites what a slower one still reads.
#define SAMPLE_SLICES 8

__device__ __forceinline__ uint32_t sc_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t sc_map(const void* p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ void sc_store(uint32_t addr, float v) { asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void sc_store(uint32_t addr, int v) { asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ void sc_sync() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}

// What the CTAs of a row tell one another, per slice; two copies, used in turn.
struct SampleExchange {
    float val[SAMPLE_SLICES];                // arg-max value / mass / kept mass of a slice
    int idx[SAMPLE_SLICES];                  // arg-max index / last kept token of a slice
    int cnt[SAMPLE_SLICES][16];              // a pass of the threshold search: tokens per digit
    float mass[SAMPLE_SLICES][16];           // ... and their mass
};

// Kept mass of a slice in vocabulary order: thread t owns the contiguous chunk [lo, hi) of the slice;
// on return excl / upto are the kept mass before and up to the end of its chunk, s_incl[last] the
// slice's kept mass and *s_last its last kept token (-1: none).
__device__ __forceinline__ void slice_scan(const float* row, int lo_s, int hi_s, uint32_t tau, float m, float inv_t, float* s_scan,
                           float* s_incl, int* s_last, int& lo, int& hi, int& last_kept, float& excl, float& upto) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int C = (hi_s - lo_s + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    lo = min(hi_s, lo_s + tid * C);
    hi = min(hi_s, lo + C);
    float local = 0.f;
    last_kept = -1;
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        if (order_key(v) >= tau && !(v != v)) { local += expf((v - m) * inv_t); last_kept = i; }
    }
    float incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    __syncthreads();                                   // the previous use of the shared arrays is over
    if (tid == 0) *s_last = -1;
    if (lane == 31) s_scan[warp] = incl;
    __syncthreads();
    if (last_kept >= 0) atomicMax(s_last, last_kept);
    if (warp == 0) {
        const int nw = SAMPLE_THREADS >> 5;
        float w = lane < nw ? s_scan[lane] : 0.f;
        float wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += n;
        }
        if (lane < nw) s_scan[lane] = wi - w;          // exclusive prefix of the warp
    }
    __syncthreads();
    // inclusive prefixes in shared memory, so that neighbouring chunks tile [0, kept mass)
    // without gaps or overlaps whatever the rounding
    s_incl[tid] = s_scan[warp] + incl;
    __syncthreads();
    excl = tid > 0 ? s_incl[tid - 1] : 0.f;
    upto = s_incl[tid];
}

// ---------------------------------------------------------------------------------------------
// The short way to the top-k / top-p threshold: three passes over the row instead of eleven.
//
// Pass 1 (arg-max) has given the row's maximum m.  Pass 2 builds ONE histogram of the row over the top
// 12 bits of the ordered bit pattern (sign, exponent, three bits of mantissa: 4,096 bins): tokens per bin
// and their mass exp((v - m) / T) as a 40-bit fixed-point integer, added with integer atomics in shared
// memory - so the sums do not depend on the order of the additions, on the number of CTAs that share the
// row or on the run.  The CTAs of a row add their bins into the first CTA's histogram through distributed
// shared memory.  From the top bin downwards the first CTA finds the bin in which the k-th token lies and
// the bin in which the cumulated mass reaches top_p x (the whole mass); the threshold lies in the higher
// of the two, and every token from that bin upwards is a candidate.  If there are at most FAST_CANDIDATES
// of them (a peaked distribution, or a small k), pass 3 gathers them - ordered bit pattern and index, in
// any order - into the first CTA's shared memory, where they are sorted (bitonic, by value then index:
// a total order, so the result is the same whatever order they arrived in), cut exactly by count and by
// cumulated mass, sorted back into vocabulary order and drawn from.  Otherwise (a flat distribution under
// top-p alone, a huge k) the kernel goes on with the general search below.
#define FAST_BINS 4096
#define FAST_CANDIDATES 2048
#define FAST_SCALE 1099511627776.0f      // 2^40

__device__ __forceinline__ void sc_red_add(uint32_t addr, unsigned int v) { asm volatile("red.shared::cluster.add.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ void sc_red_add(uint32_t addr, unsigned long long v) { asm volatile("red.shared::cluster.add.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory"); }
__device__ __forceinline__ unsigned int sc_atom_add(uint32_t addr, unsigned int v) {
    unsigned int old;
    asm volatile("atom.shared::cluster.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void sc_store(uint32_t addr, unsigned long long v) { asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory"); }
__device__ __forceinline__ float key_value(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// Bitonic sort of n_pad (a power of two, <= 2 * SAMPLE_THREADS) 64-bit keys in shared memory, descending.
__device__ void sort_desc(unsigned long long* a, int n_pad) {
    for (int k = 2; k <= n_pad; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = threadIdx.x; t < n_pad / 2; t += SAMPLE_THREADS) {
                const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1)), l = i | j;          // the pair (i, i + j)
                const bool desc = (i & k) == 0;
                const unsigned long long x = a[i], y = a[l];
                if ((x < y) == desc) { a[i] = y; a[l] = x; }
            }
            __syncthreads();
        }
}

// Inclusive sums of n (<= 2 * SAMPLE_THREADS) floats in shared memory, in place, in index order: thread t owns
// elements 2t and 2t + 1; warp scans by shuffles, warp totals through s_scan.  The same order every time.
__device__ void scan_inclusive(float* a, int n, float* s_scan) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float x0 = 2 * tid < n ? a[2 * tid] : 0.f, x1 = 2 * tid + 1 < n ? a[2 * tid + 1] : 0.f;
    float incl = x0 + x1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    __syncthreads();
    if (lane == 31) s_scan[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        float w = s_scan[lane], wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float v = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += v;
        }
        s_scan[lane] = wi - w;
    }
    __syncthreads();
    const float before = s_scan[warp] + incl - (x0 + x1);
    if (2 * tid < n) a[2 * tid] = before + x0;
    if (2 * tid + 1 < n) a[2 * tid + 1] = before + x0 + x1;
    __syncthreads();
}

struct FastShared {
    unsigned int n_cand;        // candidates gathered so far (in the first CTA)
    int go;                     // 1: the short way serves the row; 0: the general search
    int bin;                    // candidates are the tokens from this bin upwards
    int kept, pick;
    unsigned long long z_q;     // the row's whole mass, fixed point
};

// The first CTA's end of the short way: sort the gathered candidates, cut by count and by mass, draw.
__device__ void short_way_finish(unsigned long long* cand, float* cmass, float m, float inv_t, int k, float pp, bool use_k, bool use_p,
                                 unsigned long long seed, long long draw, int* out_token, float* s_scan, FastShared* fs) {
    const int tid = threadIdx.x;
    const int n = (int)min(fs->n_cand, (unsigned int)FAST_CANDIDATES);
    int n_pad = 2;
    while (n_pad < n) n_pad <<= 1;
    for (int i = n + tid; i < n_pad; i += SAMPLE_THREADS) cand[i] = 0ull;       // sorts behind every candidate
    __syncthreads();
    sort_desc(cand, n_pad);
    // masses in descending order of value and their running sums
    for (int i = tid; i < n; i += SAMPLE_THREADS) cmass[i] = expf((key_value((uint32_t)(cand[i] >> 32)) - m) * inv_t);
    __syncthreads();
    scan_inclusive(cmass, n, s_scan);
    // the threshold: the value of the k-th candidate, and of the first whose running sum reaches top_p x the whole mass
    __shared__ unsigned int s_tau_k, s_tau_p;
    if (tid == 0) {
        s_tau_k = use_k ? (uint32_t)(cand[min(k, n) - 1] >> 32) : 0u;
        s_tau_p = 0u;
    }
    __syncthreads();
    if (use_p) {
        const float target = pp * (float)((double)fs->z_q * (1.0 / (double)FAST_SCALE));
        for (int i = tid; i < n; i += SAMPLE_THREADS)
            if (cmass[i] >= target && (i == 0 || cmass[i - 1] < target)) s_tau_p = (uint32_t)(cand[i] >> 32);
    }
    __syncthreads();
    const uint32_t tau = max(s_tau_k, s_tau_p);
    // kept: the candidates whose value is at least the threshold - a prefix of the sorted list
    for (int i = tid; i < n; i += SAMPLE_THREADS)
        if ((uint32_t)(cand[i] >> 32) >= tau && (i + 1 == n || (uint32_t)(cand[i + 1] >> 32) < tau)) fs->kept = i + 1;
    __syncthreads();
    const int L = fs->kept;
    // back into vocabulary order: (index, mass bits), ascending = descending of the complement
    int l_pad = 2;
    while (l_pad < L) l_pad <<= 1;
    for (int i = tid; i < l_pad; i += SAMPLE_THREADS) {
        unsigned long long w = 0ull;
        if (i < L) {
            const uint32_t key = (uint32_t)(cand[i] >> 32), inv_idx = (uint32_t)cand[i];
            w = ((unsigned long long)inv_idx << 32) | (unsigned long long)__float_as_uint(expf((key_value(key) - m) * inv_t));
        }
        cand[i] = w;
    }
    __syncthreads();
    sort_desc(cand, l_pad);                               // descending complemented index = ascending index; padding (0) last
    for (int i = tid; i < L; i += SAMPLE_THREADS) cmass[i] = __uint_as_float((uint32_t)cand[i]);
    __syncthreads();
    scan_inclusive(cmass, L, s_scan);
    uint32_t c4[4] = {(uint32_t)(draw & 0xffffffffll), (uint32_t)((unsigned long long)draw >> 32), 0u, 0u};
    philox4x32_10(c4, (uint32_t)(seed & 0xffffffffull), (uint32_t)(seed >> 32));
    const float u = (float)(c4[0] >> 8) * (1.0f / 16777216.0f);
    const float t_draw = u * cmass[L - 1];
    for (int i = tid; i < L; i += SAMPLE_THREADS)
        if (cmass[i] > t_draw && (i == 0 || cmass[i - 1] <= t_draw)) fs->pick = i;
    __syncthreads();
    if (tid == 0) {
        const int pick = fs->pick >= 0 ? fs->pick : L - 1;           // rounding put the target at the kept mass: the last kept token
        *out_token = (int)(0xffffffffu - (uint32_t)(cand[pick] >> 32));
    }
}

// Returns true if the row has been sampled (out[r] written by the first CTA); false: go on with the general search.
__device__ bool sample_short_way(const float* __restrict__ row, int V, float m, float inv_t, int k, float pp, bool use_k, bool use_p,
                                 unsigned long long seed, long long draw, int* out_token, unsigned char* s_dyn, float* s_scan,
                                 FastShared* fs) {
    const int CL = gridDim.x, rank = (int)sc_rank(), tid = threadIdx.x;
    unsigned int* h_cnt = reinterpret_cast<unsigned int*>(s_dyn);                                   // [FAST_BINS]
    unsigned long long* h_mass = reinterpret_cast<unsigned long long*>(s_dyn + FAST_BINS * 4);      // [FAST_BINS]
    unsigned long long* cand = h_mass + FAST_BINS;                                                  // [FAST_CANDIDATES]
    float* cmass = reinterpret_cast<float*>(cand + FAST_CANDIDATES);                                // [FAST_CANDIDATES]
    for (int b = tid; b < FAST_BINS; b += SAMPLE_THREADS) { h_cnt[b] = 0u; h_mass[b] = 0ull; }
    if (tid == 0) { fs->n_cand = 0u; fs->go = 0; fs->bin = 0; fs->kept = 0; fs->pick = -1; fs->z_q = 0ull; }
    __syncthreads();
    // this CTA's share of the row
    const int per = (((V + CL - 1) / CL) + 3) & ~3;
    const int lo = min(V, rank * per), hi = min(V, lo + per);
    for (int i = lo + tid; i < hi; i += SAMPLE_THREADS) {
        const float v = row[i];
        if (v != v) continue;
        const uint32_t bin = order_key(v) >> 20;
        atomicAdd(&h_cnt[bin], 1u);
        atomicAdd(&h_mass[bin], __float2ull_rz(expf((v - m) * inv_t) * FAST_SCALE));
    }
    sc_sync();                                            // every CTA's histogram is complete (and the first CTA's is no longer being zeroed)
    if (rank != 0) {
        for (int b = tid; b < FAST_BINS; b += SAMPLE_THREADS)
            if (h_cnt[b]) { sc_red_add(sc_map(&h_cnt[b], 0), h_cnt[b]); sc_red_add(sc_map(&h_mass[b], 0), h_mass[b]); }
    }
    sc_sync();
    if (rank == 0) {
        // cumulated counts and masses from the top bin down: thread t owns the bins 4095 - 4t ... 4092 - 4t
        const int lane = tid & 31, warp = tid >> 5;
        unsigned int c_own = 0u;
        unsigned long long m_own = 0ull;
#pragma unroll
        for (int j = 0; j < 4; ++j) { c_own += h_cnt[FAST_BINS - 1 - 4 * tid - j]; m_own += h_mass[FAST_BINS - 1 - 4 * tid - j]; }
        unsigned int c_inc = c_own;
        unsigned long long m_inc = m_own;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int cv = __shfl_up_sync(0xffffffffu, c_inc, o);
            const unsigned long long mv = __shfl_up_sync(0xffffffffu, m_inc, o);
            if (lane >= o) { c_inc += cv; m_inc += mv; }
        }
        __shared__ unsigned int w_cnt[32];
        __shared__ unsigned long long w_mass[32];
        __shared__ int s_bk, s_bp;
        if (lane == 31) { w_cnt[warp] = c_inc; w_mass[warp] = m_inc; }
        if (tid == 0) { s_bk = -1; s_bp = -1; }
        __syncthreads();
        unsigned int c_before = 0u, c_total = 0u;
        unsigned long long m_before = 0ull, m_total = 0ull;
        for (int w = 0; w < 32; ++w) {
            if (w < warp) { c_before += w_cnt[w]; m_before += w_mass[w]; }
            c_total += w_cnt[w]; m_total += w_mass[w];
        }
        c_before += c_inc - c_own;
        m_before += m_inc - m_own;
        // the bin of the k-th token and the bin in which the mass reaches the target: exactly one thread finds each
        const unsigned long long target = use_p ? (unsigned long long)((double)pp * (double)m_total) : 0ull;
        unsigned int c_run = c_before;
        unsigned long long m_run = m_before;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int b = FAST_BINS - 1 - 4 * tid - j;
            const unsigned int c = h_cnt[b];
            const unsigned long long mm = h_mass[b];
            if (use_k && c_run < (unsigned int)k && c_run + c >= (unsigned int)k) s_bk = b;
            if (use_p && target > 0ull && m_run < target && m_run + mm >= target) s_bp = b;
            c_run += c; m_run += mm;
        }
        __syncthreads();
        // (fewer than k tokens, or a mass that rounding keeps below the target: that filter keeps everything)
        const bool k_on = use_k && s_bk >= 0, p_on = use_p && s_bp >= 0;
        const int bin = max(k_on ? s_bk : 0, p_on ? s_bp : 0);
        // tokens from `bin` upwards: one more pass over the cumulated counts
        __shared__ unsigned int s_n;
        if (tid == 0) s_n = 0u;
        __syncthreads();
        {
            unsigned int mine = 0u;
#pragma unroll
            for (int j = 0; j < 4; ++j) { const int b = FAST_BINS - 1 - 4 * tid - j; if (b >= bin) mine += h_cnt[b]; }
            if (mine) atomicAdd(&s_n, mine);
        }
        __syncthreads();
        const bool go = (k_on || p_on) && s_n > 0u && s_n <= FAST_CANDIDATES && c_total > 0u;
        if (tid < CL) { sc_store(sc_map(&fs->go, tid), go ? 1 : 0); sc_store(sc_map(&fs->bin, tid), bin); }
        if (tid == 0) fs->z_q = m_total;
    }
    sc_sync();
    if (!fs->go) return false;
    // ---- pass 3: the candidates go to the first CTA, (ordered bits, complemented index) in one word
    {
        const uint32_t bin = (uint32_t)fs->bin;
        const uint32_t cnt_addr = sc_map(&fs->n_cand, 0), cand_addr = sc_map(cand, 0);
        for (int i = lo + tid; i < hi; i += SAMPLE_THREADS) {
            const float v = row[i];
            if (v != v) continue;
            const uint32_t key = order_key(v);
            if ((key >> 20) >= bin) {
                const unsigned int pos = sc_atom_add(cnt_addr, 1u);
                if (pos < FAST_CANDIDATES) sc_store(cand_addr + pos * 8u, ((unsigned long long)key << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i));
            }
        }
    }
    sc_sync();
    if (rank != 0) return true;                           // the first CTA finishes the row; nobody's shared memory is touched from outside any more
    short_way_finish(cand, cmass, m, inv_t, k, pp, use_k, use_p, seed, draw, out_token, s_scan, fs);
    return true;
}

// The short way for rows with a top-k: TWO passes over the row.  Pass A finds the row's maximum (larger value, then
// lower index - the same whatever the order) and counts the tokens per bin; no exponential, no mass: the bin of the
// k-th token follows from the counts alone.  Pass B gathers the tokens from that bin upwards and adds up the row's
// whole mass as 40-bit fixed-point integers in registers (needed only for a top-p cut, which then lies among the
// candidates or below them all).  `m_out` / `best_out` carry the maximum on to the general search if there are too
// many candidates (a k beyond FAST_CANDIDATES, a huge tie).
__device__ bool sample_short_way_k(const float* __restrict__ row, int V, float inv_t, int k, float pp, bool use_p,
                                   unsigned long long seed, long long draw, int* out_token, unsigned char* s_dyn, float* s_scan,
                                   float* s_val, int* s_idx, FastShared* fs, float& m_out, int& best_out) {
    const int CL = gridDim.x, rank = (int)sc_rank(), tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned int* h_cnt = reinterpret_cast<unsigned int*>(s_dyn);                                   // [FAST_BINS]
    unsigned long long* h_mass = reinterpret_cast<unsigned long long*>(s_dyn + FAST_BINS * 4);      // (unused here; keeps the layout)
    unsigned long long* cand = h_mass + FAST_BINS;                                                  // [FAST_CANDIDATES]
    float* cmass = reinterpret_cast<float*>(cand + FAST_CANDIDATES);                                // [FAST_CANDIDATES]
    __shared__ float x_val[8];
    __shared__ int x_idx[8];
    for (int b = tid; b < FAST_BINS; b += SAMPLE_THREADS) h_cnt[b] = 0u;
    if (tid == 0) { fs->n_cand = 0u; fs->go = 0; fs->bin = 0; fs->kept = 0; fs->pick = -1; fs->z_q = 0ull; }
    __syncthreads();
    const int per = (((V + CL - 1) / CL) + 3) & ~3;
    const int lo = min(V, rank * per), hi = min(V, lo + per);
    // ---- pass A: maximum and counts
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + tid; i < hi; i += SAMPLE_THREADS) {
        const float v = row[i];
        if (v != v) continue;
        if (v > bv) { bv = v; bi = i; }                   // indices rise within a thread: a strict comparison keeps the lowest
        atomicAdd(&h_cnt[order_key(v) >> 20], 1u);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_combine(bv, bi, ov, oi);
    }
    if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = s_val[lane]; bi = s_idx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_combine(bv, bi, ov, oi);
        }
        if (lane < CL) { sc_store(sc_map(&x_val[rank], lane), bv); sc_store(sc_map(&x_idx[rank], lane), bi); }
    }
    sc_sync();                                            // maxima exchanged, every CTA's counts complete
    float m = -INFINITY;
    int best = 0x7fffffff;
    for (int c = 0; c < CL; ++c) argmax_combine(m, best, x_val[c], x_idx[c]);
    if (best == 0x7fffffff) best = 0;
    m_out = m; best_out = best;
    if (rank != 0) {
        for (int b = tid; b < FAST_BINS; b += SAMPLE_THREADS)
            if (h_cnt[b]) sc_red_add(sc_map(&h_cnt[b], 0), h_cnt[b]);
    }
    sc_sync();
    if (rank == 0) {
        // the bin of the k-th token, counted from the top bin down: thread t owns the bins 4095 - 4t ... 4092 - 4t
        unsigned int c_own = 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) c_own += h_cnt[FAST_BINS - 1 - 4 * tid - j];
        unsigned int c_inc = c_own;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int cv = __shfl_up_sync(0xffffffffu, c_inc, o);
            if (lane >= o) c_inc += cv;
        }
        __shared__ unsigned int w_cnt[32];
        __shared__ int s_bk;
        __shared__ unsigned int s_n;
        if (lane == 31) w_cnt[warp] = c_inc;
        if (tid == 0) { s_bk = -1; s_n = 0u; }
        __syncthreads();
        unsigned int c_run = c_inc - c_own;
        for (int w = 0; w < warp; ++w) c_run += w_cnt[w];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int b = FAST_BINS - 1 - 4 * tid - j;
            const unsigned int c = h_cnt[b];
            if (c_run < (unsigned int)k && c_run + c >= (unsigned int)k) { s_bk = b; s_n = c_run + c; }
            c_run += c;
        }
        __syncthreads();
        const bool go = s_bk >= 0 && s_n <= FAST_CANDIDATES;         // (fewer than k tokens in the row: the general search)
        if (tid < CL) { sc_store(sc_map(&fs->go, tid), go ? 1 : 0); sc_store(sc_map(&fs->bin, tid), s_bk); }
    }
    sc_sync();
    if (!fs->go) return false;
    // ---- pass B: candidates to the first CTA; the whole mass, if a top-p cut wants it
    {
        const uint32_t bin = (uint32_t)fs->bin;
        const uint32_t cnt_addr = sc_map(&fs->n_cand, 0), cand_addr = sc_map(cand, 0);
        unsigned long long z = 0ull;
        for (int i = lo + tid; i < hi; i += SAMPLE_THREADS) {
            const float v = row[i];
            if (v != v) continue;
            const uint32_t key = order_key(v);
            if (use_p) z += __float2ull_rz(expf((v - m) * inv_t) * FAST_SCALE);
            if ((key >> 20) >= bin) {
                const unsigned int pos = sc_atom_add(cnt_addr, 1u);
                if (pos < FAST_CANDIDATES) sc_store(cand_addr + pos * 8u, ((unsigned long long)key << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i));
            }
        }
        if (use_p) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
            if (lane == 0) sc_red_add(sc_map(&fs->z_q, 0), z);
        }
    }
    sc_sync();
    if (rank != 0) return true;
    short_way_finish(cand, cmass, m, inv_t, k, pp, true, use_p, seed, draw, out_token, s_scan, fs);
    return true;
}

__device__ int g_sample_short_way = 1;      // 0: always the general search (tests compare the two)

__global__ void __launch_bounds__(SAMPLE_THREADS, 1)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ seeds, const long long* __restrict__ draw_index,
              int* __restrict__ out, int V) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    __shared__ float s_val[33];
    __shared__ int s_idx[33];
    __shared__ float s_scan[SAMPLE_THREADS / 32 + 1];
    __shared__ int s_result, s_last;
    __shared__ float s_incl[SAMPLE_THREADS];
    __shared__ int s_cnt[2][16];
    __shared__ float s_mass[2][16];
    __shared__ SampleExchange xch[2];
    __shared__ FastShared fast_shared;
    extern __shared__ __align__(16) unsigned char s_dyn_fast[];      // the dynamic shared memory, as the short way lays it out
    // gridDim.x CTAs (1, 2, 4 or 8: the cluster) share row blockIdx.y; this one owns the slices [first, first + per)
    const int CL = gridDim.x, rank = (int)sc_rank(), tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per = SAMPLE_SLICES / CL, first = rank * per;
    const int r = blockIdx.y;
    const float* row = logits + (size_t)r * V;
    const int S = (((V + SAMPLE_SLICES - 1) / SAMPLE_SLICES) + 3) & ~3;     // slices of an aligned row start on 16-byte boundaries
    const float T = temperature ? temperature[r] : 0.f;
    int turn = 0;                                        // which copy of the exchange buffers is written next
    sc_sync();                                           // every CTA of the cluster runs before its memory is written

    const int k_row = top_k ? top_k[r] : 0;
    const float p_row = top_p ? top_p[r] : 1.0f;
    const bool uk_row = k_row > 0 && k_row < V, up_row = p_row < 1.0f;
    float m = -INFINITY;
    int best = 0x7fffffff;
    bool have_max = false;
    if (T > 0.f && uk_row && g_sample_short_way) {
        // top-k rows: maximum, counts and candidates in two passes; too many candidates: the maximum is kept, the search below goes on
        if (sample_short_way_k(row, V, 1.0f / T, k_row, p_row, up_row, seeds[r], draw_index[r], out + r, s_dyn_fast, s_scan,
                               s_val, s_idx, &fast_shared, m, best))
            return;
        have_max = true;
        sc_sync();                                       // (the first CTA's shared memory is no longer written from outside)
    }
    if (!have_max) {
    // ---- arg-max of the row
    for (int sl = first; sl < first + per; ++sl) {
        const int lo_s = min(V, sl * S), n_s = min(V, lo_s + S) - lo_s;
        int bi = lo_s;
        float bv = -INFINITY;
        if (n_s > 0) { bi = lo_s + block_argmax(row + lo_s, n_s, s_val, s_idx); bv = s_val[0]; }
        if (tid < CL) {
            sc_store(sc_map(&xch[turn].val[sl], tid), bv);
            sc_store(sc_map(&xch[turn].idx[sl], tid), bi);
        }
    }
    sc_sync();
    for (int sl = 0; sl < SAMPLE_SLICES; ++sl) argmax_combine(m, best, xch[turn].val[sl], xch[turn].idx[sl]);   // larger value, then lower index
    if (best == 0x7fffffff) best = 0;
    turn ^= 1;
    }
    if (!(T > 0.f)) {
        if (rank == 0 && tid == 0) out[r] = best;
        return;
    }
    const float inv_t = 1.0f / T;

    // ---- top-k / top-p: the short way (one histogram, then the few candidates) where it serves the row
    {
        const int k_ = k_row;
        const float p_ = p_row;
        const bool uk = uk_row, up = up_row;
        if (!uk && up && g_sample_short_way) {
            if (sample_short_way(row, V, m, inv_t, k_, p_, uk, up, seeds[r], draw_index[r], out + r, s_dyn_fast, s_scan, &fast_shared))
                return;
        }
    }

    // ---- mass of everything
    for (int sl = first; sl < first + per; ++sl) {
        const int lo_s = min(V, sl * S), hi_s = min(V, lo_s + S);
        float part = 0.f;
        for (int i = lo_s + tid; i < hi_s; i += SAMPLE_THREADS) part += expf((row[i] - m) * inv_t);
        part = rv_block_sum(part, s_val);
        if (tid < CL) sc_store(sc_map(&xch[turn].val[sl], tid), part);
    }
    sc_sync();
    float total = 0.f;
    for (int sl = 0; sl < SAMPLE_SLICES; ++sl) total += xch[turn].val[sl];
    turn ^= 1;

    // ---- threshold key: keep tokens whose order key is >= tau.  tau is the largest key c with
    // count(key >= c) >= k (top-k), or with mass(key >= c) >= top_p * total (top-p); it is found four
    // bits at a time, eight passes over the row: every thread counts its tokens (and adds their mass)
    // by the next four bits of the key in 16 slots of its own in shared memory, for the tokens that
    // agree with the bits decided so far; the block adds the slots up in a fixed order, the slices'
    // sums are added in slice order, and the largest digit that still satisfies the condition is
    // taken.  No atomics: the same result in every run.  NaN is never kept.
    uint32_t tau = 0;
    const int k = top_k ? top_k[r] : 0;
    const float pp = top_p ? top_p[r] : 1.0f;
    bool use_k = k > 0 && k < V;
    bool use_p = pp < 1.0f;
    if (use_k || use_p) {
        extern __shared__ __align__(16) unsigned char s_dyn[];
        int* h_cnt = reinterpret_cast<int*>(s_dyn);                                   // [16][SAMPLE_THREADS]
        float* h_mass = reinterpret_cast<float*>(s_dyn) + 16 * SAMPLE_THREADS;       // [16][SAMPLE_THREADS]
        uint32_t pre_k = 0, pre_p = 0;        // the bits decided so far
        int above_cnt = 0;                    // tokens whose decided bits are greater than pre_k
        float above_mass = 0.f;               // mass of the tokens whose decided bits are greater than pre_p
        const float target = pp * total;
        for (int shift = 28; shift >= 0; shift -= 4) {
            for (int sl = first; sl < first + per; ++sl) {
                const int lo_s = min(V, sl * S), hi_s = min(V, lo_s + S);
#pragma unroll
                for (int d = 0; d < 16; ++d) { h_cnt[d * SAMPLE_THREADS + tid] = 0; h_mass[d * SAMPLE_THREADS + tid] = 0.f; }
                // four loads in flight per thread
                for (int i0 = lo_s + tid; i0 < hi_s; i0 += 4 * SAMPLE_THREADS) {
                    float vs[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int i = i0 + j * SAMPLE_THREADS;
                        vs[j] = i < hi_s ? row[i] : __int_as_float(0x7fc00000);      // NaN: skipped below
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float v = vs[j];
                        if (v != v) continue;
                        const uint32_t key = order_key(v);
                        const int d = (int)((key >> shift) & 15u);
                        const bool top = shift == 28;
                        if (use_k && (top || (key >> (shift + 4)) == (pre_k >> (shift + 4)))) h_cnt[d * SAMPLE_THREADS + tid] += 1;
                        if (use_p && (top || (key >> (shift + 4)) == (pre_p >> (shift + 4)))) h_mass[d * SAMPLE_THREADS + tid] += expf((v - m) * inv_t);
                    }
                }
                __syncthreads();
                {   // warp w adds digit w % 16 over one half of the threads, lanes in a fixed order
                    const int d = warp & 15, half = warp >> 4;
                    int c = 0;
                    float ms = 0.f;
                    for (int j = lane; j < SAMPLE_THREADS / 2; j += 32) {
                        c += h_cnt[d * SAMPLE_THREADS + half * (SAMPLE_THREADS / 2) + j];
                        ms += h_mass[d * SAMPLE_THREADS + half * (SAMPLE_THREADS / 2) + j];
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        c += __shfl_xor_sync(0xffffffffu, c, o);
                        ms += __shfl_xor_sync(0xffffffffu, ms, o);
                    }
                    if (lane == 0) { s_cnt[half][d] = c; s_mass[half][d] = ms; }
                }
                __syncthreads();
                // this slice's 16 + 16 sums go to every CTA of the row
                if (tid < 16 * CL) {
                    const int d = tid & 15, to = tid >> 4;
                    sc_store(sc_map(&xch[turn].cnt[sl][d], to), s_cnt[0][d] + s_cnt[1][d]);
                    sc_store(sc_map(&xch[turn].mass[sl][d], to), s_mass[0][d] + s_mass[1][d]);
                }
            }
            sc_sync();
            // every thread of every CTA takes the same decision from the same sums
            if (use_k) {
                int run = above_cnt, found = -1;
                for (int d = 15; d >= 0; --d) {
                    int c = 0;
                    for (int sl = 0; sl < SAMPLE_SLICES; ++sl) c += xch[turn].cnt[sl][d];
                    if (run + c >= k) { found = d; break; }
                    run += c;
                }
                if (found < 0) { use_k = false; pre_k = 0; }          // fewer than k tokens (NaN rows): keep all
                else { pre_k |= (uint32_t)found << shift; above_cnt = run; }
            }
            if (use_p) {
                float run = above_mass;
                int found = -1;
                for (int d = 15; d >= 0; --d) {
                    float c = 0.f;
                    for (int sl = 0; sl < SAMPLE_SLICES; ++sl) c += xch[turn].mass[sl][d];
                    if (run + c >= target) { found = d; break; }
                    run += c;
                }
                if (found < 0) { use_p = false; pre_p = 0; }          // rounding left the sum just below the target: keep all
                else { pre_p |= (uint32_t)found << shift; above_mass = run; }
            }
            turn ^= 1;
            if (!use_k && !use_p) break;
        }
        tau = pre_k > pre_p ? pre_k : pre_p;
    }

    // ---- kept mass and last kept token of every slice, to every CTA
    int lo, hi, last_kept;
    float excl, upto;
    for (int sl = first; sl < first + per; ++sl) {
        const int lo_s = min(V, sl * S), hi_s = min(V, lo_s + S);
        slice_scan(row, lo_s, hi_s, tau, m, inv_t, s_scan, s_incl, &s_last, lo, hi, last_kept, excl, upto);
        if (tid < CL) {
            sc_store(sc_map(&xch[turn].val[sl], tid), s_incl[SAMPLE_THREADS - 1]);
            sc_store(sc_map(&xch[turn].idx[sl], tid), s_last);
        }
    }
    sc_sync();
    float kept_total = 0.f;
    for (int sl = 0; sl < SAMPLE_SLICES; ++sl) kept_total += xch[turn].val[sl];

    // ---- the draw: the first token, in vocabulary order, whose cumulated kept mass exceeds u * (kept mass)
    uint32_t c4[4] = {(uint32_t)(draw_index[r] & 0xffffffffll), (uint32_t)((unsigned long long)draw_index[r] >> 32), 0u, 0u};
    philox4x32_10(c4, (uint32_t)(seeds[r] & 0xffffffffull), (uint32_t)(seeds[r] >> 32));
    const float u = (float)(c4[0] >> 8) * (1.0f / 16777216.0f);
    const float target = u * kept_total;
    // the slice the target falls into (the same arithmetic in every CTA); if rounding put the target at
    // or beyond the kept mass, the slice of the last kept token
    int resp = -1;
    float off = 0.f, resp_off = 0.f;
    for (int sl = 0; sl < SAMPLE_SLICES; ++sl) {
        const float kc = xch[turn].val[sl];
        if (resp < 0 && kc > 0.f && target < off + kc) { resp = sl; resp_off = off; }
        off += kc;
    }
    bool beyond = false;
    if (resp < 0) {
        beyond = true;
        for (int sl = SAMPLE_SLICES - 1; sl >= 0; --sl)
            if (xch[turn].idx[sl] >= 0) { resp = sl; break; }
    }
    if (resp < 0) {                                       // nothing was kept at all (a row of NaN): the arg-max
        if (rank == 0 && tid == 0) out[r] = best;
        return;
    }
    if (resp / per != rank) return;                       // (nothing of another CTA is touched after the barrier above)
    {
        const int lo_s = min(V, resp * S), hi_s = min(V, lo_s + S);
        slice_scan(row, lo_s, hi_s, tau, m, inv_t, s_scan, s_incl, &s_last, lo, hi, last_kept, excl, upto);
        if (tid == 0) s_result = -1;
        __syncthreads();
        const float t_loc = target - resp_off;
        if (!beyond && upto > excl && excl <= t_loc && t_loc < upto) {
            float run = excl;
            int pick = last_kept;
            for (int i = lo; i < hi; ++i) {
                const float v = row[i];
                if (order_key(v) >= tau && !(v != v)) {
                    run += expf((v - m) * inv_t);
                    if (run > t_loc) { pick = i; break; }
                }
            }
            atomicMax(&s_result, pick);   // at most one thread matches; max is only a tie guard
        }
        __syncthreads();
        // no chunk took it (rounding): the last kept token of the slice
        if (tid == 0) out[r] = s_result >= 0 ? s_result : (s_last >= 0 ? s_last : best);
    }
}

static int g_sample_cluster = 0;
// CTAs per row: 0 chosen by the number of rows, else 1, 2, 4 or 8 (for tests: the result is the same).
RV_EXPORT void rv_sample_set_cluster(int ctas_per_row) { g_sample_cluster = ctas_per_row; }
// 1 (default): top-k / top-p rows try the short way first; 0: always the general search.
RV_EXPORT int rv_sample_set_short_way(int on) {
    const int v = on ? 1 : 0;
    return (int)cudaMemcpyToSymbol(g_sample_short_way, &v, sizeof(int));
}

// temperature, top_k, top_p may be null (greedy / disabled).  seeds and draw_index are read
// only for rows with temperature > 0.
RV_EXPORT int rv_sample(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                        const unsigned long long* seeds, const long long* draw_index, int* out,
                        int n_rows, int vocab, cudaStream_t stream) {
    if (n_rows < 0 || vocab <= 0) return RV_ERR_BAD_SIZE;
    if (n_rows == 0) return RV_OK;
    if (temperature && (!seeds || !draw_index)) return RV_ERR_BAD_SIZE;
    // the threshold search of top-k / top-p keeps 16 counters and 16 sums per thread in shared memory
    const size_t smem = (temperature && (top_k || top_p)) ? (size_t)2 * 16 * SAMPLE_THREADS * 4 : 0;
    static RvPerDevice configured;
    if (smem) {
        if (int e = rv_configure_smem(configured, sample_kernel, (int)(2 * 16 * SAMPLE_THREADS * 4))) return e;
    }
    if (n_rows > 65535) return RV_ERR_BAD_SIZE;
    // CTAs per row: as many (8, 4, 2 or 1) as keep rows x CTAs within the SMs; the result is the same for each
    const int sms = rv_sm_count();
    int cl = g_sample_cluster > 0 ? g_sample_cluster : (n_rows * 8 <= sms ? 8 : (n_rows * 4 <= sms ? 4 : (n_rows * 2 <= sms ? 2 : 1)));
    if (cl != 1 && cl != 2 && cl != 4 && cl != 8) return RV_ERR_BAD_SIZE;
    RV_LAUNCH_ST = rv_launch_cluster(sample_kernel, dim3(cl, n_rows), dim3(SAMPLE_THREADS), smem, stream, (unsigned)cl,
                                     logits, temperature, top_k, top_p, seeds, draw_index, out, vocab);
    return rv_launch_status();
}
