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
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
        const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
        c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
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

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ seeds, const long long* __restrict__ draw_index,
              int* __restrict__ out, int V) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    __shared__ float s_val[33];
    __shared__ int s_idx[33];
    __shared__ float s_scan[SAMPLE_THREADS / 32 + 1];
    __shared__ int s_result;
    __shared__ float s_incl[SAMPLE_THREADS];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * V;
    const float T = temperature ? temperature[r] : 0.f;
    const int best = block_argmax(row, V, s_val, s_idx);
    if (!(T > 0.f)) {
        if (threadIdx.x == 0) out[r] = best;
        return;
    }
    const float m = s_val[0];
    const float inv_t = 1.0f / T;
    __syncthreads();

    // mass of everything
    float part = 0.f;
    if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        const float4* r4 = reinterpret_cast<const float4*>(row);
        float p1 = 0.f;
        // (four loads in flight per thread; every thread adds its elements in the same order as before)
        for (int i0 = threadIdx.x; i0 < (V >> 2); i0 += 4 * blockDim.x) {
            float4 a[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = i0 + j * blockDim.x;
                a[j] = i < (V >> 2) ? r4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (i0 + j * (int)blockDim.x >= (V >> 2)) break;
                part += expf((a[j].x - m) * inv_t) + expf((a[j].y - m) * inv_t);
                p1 += expf((a[j].z - m) * inv_t) + expf((a[j].w - m) * inv_t);
            }
        }
        part += p1;
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) part += expf((row[i] - m) * inv_t);
    }
    const float total = rv_block_sum(part, s_val);

    // threshold key: keep tokens whose order key is >= tau.  tau is the largest key c with
    // count(key >= c) >= k (top-k), or with mass(key >= c) >= top_p * total (top-p); it is found
    // four bits at a time, eight passes over the row: every thread counts its tokens (and adds
    // their mass) by the next four bits of the key in 16 slots of its own in shared memory, for the
    // tokens that agree with the bits decided so far; the block adds the slots up in a fixed order
    // and takes the largest digit that still satisfies the condition.  NaN is never kept.
    uint32_t tau = 0;
    const int k = top_k ? top_k[r] : 0;
    const float pp = top_p ? top_p[r] : 1.0f;
    bool use_k = k > 0 && k < V;
    bool use_p = pp < 1.0f;
    if (use_k || use_p) {
        extern __shared__ __align__(16) unsigned char s_dyn[];
        int* h_cnt = reinterpret_cast<int*>(s_dyn);                                   // [16][SAMPLE_THREADS]
        float* h_mass = reinterpret_cast<float*>(s_dyn) + 16 * SAMPLE_THREADS;       // [16][SAMPLE_THREADS]
        __shared__ int s_cnt[2][16];
        __shared__ float s_mass[2][16];
        const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
        uint32_t pre_k = 0, pre_p = 0;        // the bits decided so far
        int above_cnt = 0;                    // tokens whose decided bits are greater than pre_k
        float above_mass = 0.f;               // mass of the tokens whose decided bits are greater than pre_p
        const float target = pp * total;
        for (int shift = 28; shift >= 0; shift -= 4) {
#pragma unroll
            for (int d = 0; d < 16; ++d) { h_cnt[d * SAMPLE_THREADS + tid] = 0; h_mass[d * SAMPLE_THREADS + tid] = 0.f; }
            // eight loads in flight per thread: one block reads the row at the speed its loads in flight allow
            for (int i0 = tid; i0 < V; i0 += 8 * SAMPLE_THREADS) {
                float vs[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int i = i0 + j * SAMPLE_THREADS;
                    vs[j] = i < V ? row[i] : __int_as_float(0x7fc00000);      // NaN: skipped below
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
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
                const int d = warp & 15, part = warp >> 4;
                int c = 0;
                float ms = 0.f;
                for (int j = lane; j < SAMPLE_THREADS / 2; j += 32) {
                    c += h_cnt[d * SAMPLE_THREADS + part * (SAMPLE_THREADS / 2) + j];
                    ms += h_mass[d * SAMPLE_THREADS + part * (SAMPLE_THREADS / 2) + j];
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    c += __shfl_xor_sync(0xffffffffu, c, o);
                    ms += __shfl_xor_sync(0xffffffffu, ms, o);
                }
                if (lane == 0) { s_cnt[part][d] = c; s_mass[part][d] = ms; }
            }
            __syncthreads();
            // every thread takes the same decision from the same sums
            if (use_k) {
                int run = above_cnt, found = -1;
                for (int d = 15; d >= 0; --d) {
                    const int c = s_cnt[0][d] + s_cnt[1][d];
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
                    const float c = s_mass[0][d] + s_mass[1][d];
                    if (run + c >= target) { found = d; break; }
                    run += c;
                }
                if (found < 0) { use_p = false; pre_p = 0; }          // rounding left the sum just below the target: keep all
                else { pre_p |= (uint32_t)found << shift; above_mass = run; }
            }
            if (!use_k && !use_p) break;
        }
        tau = pre_k > pre_p ? pre_k : pre_p;
    }

    // inverse CDF in vocabulary order: thread t owns the contiguous chunk [t*C, (t+1)*C)
    const int C = (V + blockDim.x - 1) / blockDim.x;
    const int lo = threadIdx.x * C;
    const int hi = min(V, lo + C);
    float local = 0.f;
    int last_kept = -1;
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        if (order_key(v) >= tau && !(v != v)) { local += expf((v - m) * inv_t); last_kept = i; }
    }
    // exclusive scan of `local` over the block
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    if (threadIdx.x == 0) s_result = -1;
    __syncthreads();
    if (lane == 31) s_scan[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
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
    s_incl[threadIdx.x] = s_scan[warp] + incl;
    __syncthreads();
    const float excl = threadIdx.x > 0 ? s_incl[threadIdx.x - 1] : 0.f;
    const float upto = s_incl[threadIdx.x];
    const float kept_total = s_incl[blockDim.x - 1];

    uint32_t c[4] = {(uint32_t)(draw_index[r] & 0xffffffffll), (uint32_t)((unsigned long long)draw_index[r] >> 32), 0u, 0u};
    philox4x32_10(c, (uint32_t)(seeds[r] & 0xffffffffull), (uint32_t)(seeds[r] >> 32));
    const float u = (float)(c[0] >> 8) * (1.0f / 16777216.0f);
    const float target = u * kept_total;

    if (upto > excl && excl <= target && target < upto) {
        float run = excl;
        int pick = last_kept;
        for (int i = lo; i < hi; ++i) {
            const float v = row[i];
            if (order_key(v) >= tau && !(v != v)) {
                run += expf((v - m) * inv_t);
                if (run > target) { pick = i; break; }
            }
        }
        atomicMax(&s_result, pick);   // at most one thread matches; max is only a tie guard
    }
    __syncthreads();
    if (s_result < 0) {
        // rounding put the target at or beyond the kept mass: take the last kept token
        atomicMax(&s_result, last_kept);
        __syncthreads();
    }
    if (threadIdx.x == 0) out[r] = s_result >= 0 ? s_result : best;
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
    static bool configured = false;
    if (smem && !configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * 16 * SAMPLE_THREADS * 4));
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    RV_LAUNCH_ST = rv_launch(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), smem, stream, logits, temperature, top_k, top_p, seeds, draw_index, out, vocab);
    return rv_launch_status();
}
