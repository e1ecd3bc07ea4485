// Plain paged attention: the reference kernel that every faster attention kernel is checked
// against, and the kernel of the float32 path.  One warp per (token, query head); keys are
// walked one by one through the block table with an online softmax in float.
//
// Rule (v3/kernels/paged_attention_sm89.cu:241-369 of the reference): the q_len tokens a
// sequence brings to a step are the tail of its ctx_len cached tokens.  The token with
// in-step index i sits at position p = ctx_len - q_len + i and sees keys [0, p]; with a
// window of W keys it sees (p - W, p].  kv_head = head * nkv / nh.  A decoded token is the
// case q_len = 1.  ctx_len <= 0 marks a padded row: zeros are written, no table is read.
//
// Cache layer layout: [num_pages, 2 (k, v), nkv, page_size, hd].
#include "common.cuh"

#define MAX_DIMS_PER_LANE 8   // head_dim <= 256

template <typename T>
__global__ void paged_attention_ref_kernel(const T* __restrict__ q, const T* __restrict__ cache,
                                           const int* __restrict__ block_tables, const int* __restrict__ cu_seqlens,
                                           const int* __restrict__ ctx_lens, const int* __restrict__ token_seq,
                                           T* __restrict__ out, int n_tokens, int nh, int nkv, int hd,
                                           int page_size, int max_blocks, float scale, int window) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int t = blockIdx.x;
    const int h = blockIdx.y * (blockDim.x >> 5) + warp;
    if (h >= nh || t >= n_tokens) return;
    const int seq = token_seq[t];
    T* o = out + ((size_t)t * nh + h) * hd;
    const int ctx = seq >= 0 ? ctx_lens[seq] : 0;
    if (ctx <= 0) {
        for (int d = lane; d < hd; d += 32) o[d] = rv_from_float<T>(0.f);
        return;
    }
    const int q_start = cu_seqlens[seq];
    const int q_len = cu_seqlens[seq + 1] - q_start;
    const int pos = ctx - q_len + (t - q_start);
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int kvh = (int)(((long long)h * nkv) / nh);

    float qv[MAX_DIMS_PER_LANE], acc[MAX_DIMS_PER_LANE];
    const T* qp = q + ((size_t)t * nh + h) * hd;
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < hd ? rv_to_float(qp[d]) * scale : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int* table = block_tables + (size_t)seq * max_blocks;
    const size_t page_stride = (size_t)2 * nkv * page_size * hd;
    const size_t v_off = (size_t)nkv * page_size * hd;
    for (int j = lo; j <= pos; ++j) {
        const int page = table[j / page_size];
        const T* kp = cache + (size_t)page * page_stride + ((size_t)kvh * page_size + (j % page_size)) * hd;
        const T* vp = kp + v_off;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) s = fmaf(qv[i], rv_to_float(kp[d]), s);
        }
        s = rv_warp_sum(s);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);     // exp(-inf) = 0 at the first key
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) acc[i] = acc[i] * corr + p * rv_to_float(vp[d]);
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) o[d] = rv_from_float<T>(acc[i] * inv);
    }
}

RV_EXPORT int rv_paged_attention_ref(const void* q, const void* cache, const int* block_tables,
                                     const int* cu_seqlens, const int* ctx_lens, const int* token_seq,
                                     void* out, int n_tokens, int nh, int nkv, int hd, int page_size,
                                     int max_blocks, float scale, int window, int dtype, cudaStream_t stream) {
    if (n_tokens < 0 || nh <= 0 || nkv <= 0 || hd <= 0 || page_size <= 0 || max_blocks <= 0) return RV_ERR_BAD_SIZE;
    if (hd > 32 * MAX_DIMS_PER_LANE) return RV_ERR_UNSUPPORTED;
    if (n_tokens == 0) return RV_OK;
    const int warps = 4;
    const dim3 grid(n_tokens, (nh + warps - 1) / warps);
    if (dtype == RV_DTYPE_F32)
        RV_LAUNCH_ST = rv_launch(paged_attention_ref_kernel<float>, dim3(grid), dim3(warps * 32), 0, stream, 
            (const float*)q, (const float*)cache, block_tables, cu_seqlens, ctx_lens, token_seq, (float*)out,
            n_tokens, nh, nkv, hd, page_size, max_blocks, scale, window);
    else if (dtype == RV_DTYPE_BF16)
        RV_LAUNCH_ST = rv_launch(paged_attention_ref_kernel<__nv_bfloat16>, dim3(grid), dim3(warps * 32), 0, stream, 
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_tables, cu_seqlens, ctx_lens, token_seq,
            (__nv_bfloat16*)out, n_tokens, nh, nkv, hd, page_size, max_blocks, scale, window);
    else
        return RV_ERR_BAD_DTYPE;
    return rv_launch_status();
}
