// Row-wise kernels of the dense decoder: embedding gather, RMSNorm, rotary position
// encoding fused with the q/k/v bias and the paged cache write, and SiLU-gated product.
// All arithmetic is in float; storage is float or bfloat16.  Any row width is accepted.
//
// Formulas (paths inside the reference project):
//   gather   kernels/embedding_gather_f16.cu:12-39          (row copy, out-of-range id -> zeros)
//   rmsnorm  kernels/fused_rmsnorm_fp8_quant.cu:61-84        (x * rsqrt(mean(x^2) + eps) * gamma)
//   rotary   v3/crates/rvllm-fused/src/reference.rs:177-203  (pairs i, i + head_dim/2)
//   cache    v3/kernels/fused_rope_cache_fp8kv.cu:63-80      (slot < 0 is a padded row: skipped)
//   silu     kernels/fused_silu_fp8_quant.cu:52-56           (row = gate | up; g / (1 + e^-g) * u)
#include "common.cuh"

// ------------------------------------------------------------------ embedding / row gather
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                   T* __restrict__ out, int width, int rows_in_table) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < rows_in_table;
    const T* src = table + (size_t)(ok ? id : 0) * width;
    T* dst = out + (size_t)t * width;
    const bool vec = ((width * sizeof(T)) % 16 == 0) &&
                     ((reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(out)) % 16 == 0);
    if (vec) {
        const int n16 = width * sizeof(T) / 16;
        const uint4* s = reinterpret_cast<const uint4*>(src);
        uint4* d = reinterpret_cast<uint4*>(dst);
        for (int i = threadIdx.x; i < n16; i += blockDim.x) d[i] = ok ? s[i] : make_uint4(0, 0, 0, 0);
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = ok ? src[i] : rv_from_float<T>(0.f);
    }
}

RV_EXPORT int rv_gather_rows(const void* table, const int* ids, void* out, int n_rows, int width,
                             int rows_in_table, int dtype, cudaStream_t stream) {
    if (n_rows < 0 || width <= 0 || rows_in_table <= 0) return RV_ERR_BAD_SIZE;
    if (n_rows == 0) return RV_OK;
    const int threads = width >= 2048 ? 256 : 128;
    if (dtype == RV_DTYPE_F32)
        RV_LAUNCH_ST = rv_launch(gather_rows_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (const float*)table, ids, (float*)out, width, rows_in_table);
    else if (dtype == RV_DTYPE_BF16)
        RV_LAUNCH_ST = rv_launch(gather_rows_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, (const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out, width, rows_in_table);
    else
        return RV_ERR_BAD_DTYPE;
    return rv_launch_status();
}

// ------------------------------------------------------------------ tokens that arrive late
// A decode step can be launched before the host has read the ids that the previous step sampled:
// its one-token sequences then take their token from the previous step's output on the device.
// Sequence i with source[i] >= 0 gets token_ids[cu_seqlens[i]] = sampled[source[i]].
__global__ void late_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ cu_seqlens,
                                   const int* __restrict__ source, const int* __restrict__ sampled,
                                   int n_seqs, int n_sampled) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_seqs) return;
    const int j = source[i];
    if (j >= 0 && j < n_sampled) token_ids[cu_seqlens[i]] = sampled[j];
}

RV_EXPORT int rv_late_tokens(int* token_ids, const int* cu_seqlens, const int* source, const int* sampled,
                             int n_seqs, int n_sampled, cudaStream_t stream) {
    if (n_seqs < 0 || n_sampled < 0) return RV_ERR_BAD_SIZE;
    if (n_seqs == 0) return RV_OK;
    late_tokens_kernel<<<(n_seqs + 127) / 128, 128, 0, stream>>>(token_ids, cu_seqlens, source, sampled, n_seqs, n_sampled);
    return rv_launch_status();
}

// ------------------------------------------------------------------ RMSNorm
// One block per row.  The row is read twice (the second read hits L1/L2); the sum of squares,
// the reciprocal root and the product with gamma are formed in float and rounded once.
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const void* __restrict__ gamma, int gamma_dtype,
                               T* __restrict__ out, int width, float eps) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    __shared__ float scratch[33];
    const T* row = x + (size_t)blockIdx.x * width;
    T* dst = out + (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = rv_to_float(row[i]);
        ss = fmaf(v, v, ss);
    }
    ss = rv_block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = rv_to_float(row[i]);
        dst[i] = rv_from_float<T>(v * r * rv_load_param(gamma, gamma_dtype, i));
    }
}

// bfloat16 rows whose width is a multiple of 8: every thread keeps its 16-byte pieces of the row
// in registers, so the row is read from memory once.
template <int VPT>
__global__ void rmsnorm_bf16_vec_kernel(const __nv_bfloat16* __restrict__ x, const void* __restrict__ gamma,
                                        int gamma_dtype, __nv_bfloat16* __restrict__ out, int width, float eps) {
    rv_pdl_launch_dependents();
    __shared__ float scratch[33];
    const int nvec = width >> 3;
    // gamma is a weight: it is fetched before the wait for the kernel that writes x, 16 or 32 bytes
    // at a time where its address allows
    float g[VPT][8];
    const bool g_vec = (reinterpret_cast<uintptr_t>(gamma) & 15) == 0;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c >= nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) g[i][j] = 0.f;
        } else if (g_vec && gamma_dtype == RV_DTYPE_BF16) {
            const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gamma) + c);
            const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(gh[j]);
                g[i][2 * j] = f.x; g[i][2 * j + 1] = f.y;
            }
        } else if (g_vec && gamma_dtype == RV_DTYPE_F32) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c);
            const float4 b = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c + 1);
            g[i][0] = a.x; g[i][1] = a.y; g[i][2] = a.z; g[i][3] = a.w;
            g[i][4] = b.x; g[i][5] = b.y; g[i][6] = b.z; g[i][7] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) g[i][j] = rv_load_param(gamma, gamma_dtype, c * 8 + j);
        }
    }
    rv_pdl_wait();
    const uint4* row = reinterpret_cast<const uint4*>(x + (size_t)blockIdx.x * width);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * width);
    uint4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        v[i] = c < nvec ? row[c] : make_uint4(0, 0, 0, 0);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            ss = fmaf(f.x, f.x, ss);
            ss = fmaf(f.y, f.y, ss);
        }
    }
    ss = rv_block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c >= nvec) continue;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            oh[j] = __floats2bfloat162_rn(f.x * r * g[i][2 * j], f.y * r * g[i][2 * j + 1]);
        }
        dst[c] = o;
    }
}

RV_EXPORT int rv_rmsnorm(const void* x, const void* gamma, int gamma_dtype, void* out, int n_rows,
                         int width, float eps, int dtype, cudaStream_t stream) {
    if (n_rows < 0 || width <= 0) return RV_ERR_BAD_SIZE;
    if (n_rows == 0) return RV_OK;
    if (dtype == RV_DTYPE_BF16 && width % 8 == 0 && width <= 8 * 4 * 1024 &&
        (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) % 16 == 0) {
        const int nvec = width / 8;
        int threads = 32;
        while (threads < 256 && threads < nvec) threads <<= 1;
        while (threads < 1024 && threads * 4 < nvec) threads <<= 1;
        const int vpt = (nvec + threads - 1) / threads;
        const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
        __nv_bfloat16* op = (__nv_bfloat16*)out;
        if (vpt <= 1) RV_LAUNCH_ST = rv_launch(rmsnorm_bf16_vec_kernel<1>, dim3(n_rows), dim3(threads), 0, stream, xp, gamma, gamma_dtype, op, width, eps);
        else if (vpt <= 2) RV_LAUNCH_ST = rv_launch(rmsnorm_bf16_vec_kernel<2>, dim3(n_rows), dim3(threads), 0, stream, xp, gamma, gamma_dtype, op, width, eps);
        else RV_LAUNCH_ST = rv_launch(rmsnorm_bf16_vec_kernel<4>, dim3(n_rows), dim3(threads), 0, stream, xp, gamma, gamma_dtype, op, width, eps);
        return rv_launch_status();
    }
    int threads = 32;
    while (threads < 1024 && threads * 4 < width) threads <<= 1;
    if (dtype == RV_DTYPE_F32)
        RV_LAUNCH_ST = rv_launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (const float*)x, gamma, gamma_dtype, (float*)out, width, eps);
    else if (dtype == RV_DTYPE_BF16)
        RV_LAUNCH_ST = rv_launch(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, (const __nv_bfloat16*)x, gamma, gamma_dtype, (__nv_bfloat16*)out, width, eps);
    else
        return RV_ERR_BAD_DTYPE;
    return rv_launch_status();
}

// ------------------------------------------------------------------ rotary + bias + cache write
// qkv row layout: [q (nh*hd) | k (nkv*hd) | v (nkv*hd)].  Grid (T, nh + 2*nkv): one block per
// (token, head).  q heads: add bias, rotate, write to q_out [T, nh*hd].  k heads: add bias,
// rotate, write into the page of the token's slot.  v heads: add bias, write into the page.
// Cache layer layout: [num_pages, 2 (k, v), nkv, page_size, hd].
// cos/sin: float [table_rows, rot/2]; null pointers mean "no rotation".  `rot` <= hd is the number
// of leading elements of a head that are rotated, in pairs (i, i + rot/2); the rest of the head
// passes through (with its bias).  With write_kv = 0 the rows hold q alone (row_stride = nh*hd)
// and nothing is written to the cache.
template <typename T, typename TIn = T>
__global__ void rope_cache_write_kernel(const TIn* __restrict__ qkv, const void* __restrict__ bias, int bias_dtype,
                                        const int* __restrict__ positions, const float* __restrict__ cos_t,
                                        const float* __restrict__ sin_t, const int* __restrict__ slot_mapping,
                                        T* __restrict__ cache, T* __restrict__ q_out, int nh, int nkv, int hd,
                                        int page_size, int write_kv, int table_rows, int row_stride, int rot) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int t = blockIdx.x;
    const int head = blockIdx.y;
    const int half = rot >> 1;
    const TIn* src = qkv + (size_t)t * row_stride + (size_t)head * hd;
    const int col0 = head * hd;
    int pos = positions[t];
    if (pos < 0) pos = 0;
    if (pos >= table_rows) pos = table_rows - 1;   // the host refuses such positions; never read outside
    const bool is_q = head < nh;
    const bool is_k = !is_q && head < nh + nkv;
    T* dst;
    if (is_q) {
        dst = q_out + (size_t)t * nh * hd + (size_t)head * hd;
    } else {
        if (!write_kv) return;
        const int slot = slot_mapping[t];
        if (slot < 0) return;
        const int kvh = is_k ? head - nh : head - nh - nkv;
        const int page = slot / page_size, off = slot - page * page_size;
        dst = cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + off) * hd;
    }
    if (is_q || is_k) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float a = rv_to_float(src[i]);
            float b = rv_to_float(src[i + half]);
            if (bias) {
                a += rv_load_param(bias, bias_dtype, col0 + i);
                b += rv_load_param(bias, bias_dtype, col0 + i + half);
            }
            float c = 1.f, s = 0.f;
            if (cos_t) {
                c = cos_t[(size_t)pos * half + i];
                s = sin_t[(size_t)pos * half + i];
            }
            dst[i] = rv_from_float<T>(a * c - b * s);
            dst[i + half] = rv_from_float<T>(a * s + b * c);
        }
        for (int i = rot + threadIdx.x; i < hd; i += blockDim.x) {       // the part of the head that is not rotated
            float a = rv_to_float(src[i]);
            if (bias) a += rv_load_param(bias, bias_dtype, col0 + i);
            dst[i] = rv_from_float<T>(a);
        }
    } else {
        for (int i = threadIdx.x; i < hd; i += blockDim.x) {
            float a = rv_to_float(src[i]);
            if (bias) a += rv_load_param(bias, bias_dtype, col0 + i);
            dst[i] = rv_from_float<T>(a);
        }
    }
}

// bfloat16 with head_dim a multiple of 16: one block per token walks all heads of the row with
// 16-byte loads (8 rotation pairs at a time: 8 elements of the first half, 8 of the second).
__global__ void rope_cache_write_bf16_vec_kernel(const __nv_bfloat16* __restrict__ qkv, const void* __restrict__ bias,
                                                 int bias_dtype, const int* __restrict__ positions,
                                                 const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                 const int* __restrict__ slot_mapping, __nv_bfloat16* __restrict__ cache,
                                                 __nv_bfloat16* __restrict__ q_out, int nh, int nkv, int hd, int page_size,
                                                 int write_kv, int table_rows, int row_stride) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int t = blockIdx.x;
    const int half = hd >> 1;
    const int vec_half = half >> 3;                 // 16-byte pieces per half head
    int pos = positions[t];
    if (pos < 0) pos = 0;
    if (pos >= table_rows) pos = table_rows - 1;
    const int slot = write_kv ? slot_mapping[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot - page * page_size : 0;
    const int n_rot_heads = write_kv ? nh + nkv : nh;
    const __nv_bfloat16* row = qkv + (size_t)t * row_stride;
    // rotated heads (q, then k)
    for (int item = threadIdx.x; item < n_rot_heads * vec_half; item += blockDim.x) {
        const int head = item / vec_half, c = item - head * vec_half;
        __nv_bfloat16* dst;
        if (head < nh) {
            dst = q_out + (size_t)t * nh * hd + (size_t)head * hd;
        } else {
            if (slot < 0) continue;
            dst = cache + ((((size_t)page * 2) * nkv + (head - nh)) * page_size + off) * hd;
        }
        const __nv_bfloat16* src = row + (size_t)head * hd;
        const uint4 av = *reinterpret_cast<const uint4*>(src + c * 8);
        const uint4 bv = *reinterpret_cast<const uint4*>(src + half + c * 8);
        const __nv_bfloat16* ae = reinterpret_cast<const __nv_bfloat16*>(&av);
        const __nv_bfloat16* be = reinterpret_cast<const __nv_bfloat16*>(&bv);
        uint4 oa, ob;
        __nv_bfloat16* oae = reinterpret_cast<__nv_bfloat16*>(&oa);
        __nv_bfloat16* obe = reinterpret_cast<__nv_bfloat16*>(&ob);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = c * 8 + j;
            float a = __bfloat162float(ae[j]), b = __bfloat162float(be[j]);
            if (bias) {
                a += rv_load_param(bias, bias_dtype, head * hd + i);
                b += rv_load_param(bias, bias_dtype, head * hd + i + half);
            }
            float cs = 1.f, sn = 0.f;
            if (cos_t) { cs = cos_t[(size_t)pos * half + i]; sn = sin_t[(size_t)pos * half + i]; }
            oae[j] = __float2bfloat16_rn(a * cs - b * sn);
            obe[j] = __float2bfloat16_rn(a * sn + b * cs);
        }
        *reinterpret_cast<uint4*>(dst + c * 8) = oa;
        *reinterpret_cast<uint4*>(dst + half + c * 8) = ob;
    }
    // value heads: bias only
    if (write_kv && slot >= 0) {
        const int vec_head = hd >> 3;
        for (int item = threadIdx.x; item < nkv * vec_head; item += blockDim.x) {
            const int head = item / vec_head, c = item - head * vec_head;
            const int col0 = (nh + nkv + head) * hd;
            uint4 v = *reinterpret_cast<const uint4*>(row + col0 + c * 8);
            if (bias) {
                __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&v);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    e[j] = __float2bfloat16_rn(__bfloat162float(e[j]) + rv_load_param(bias, bias_dtype, col0 + c * 8 + j));
            }
            __nv_bfloat16* dst = cache + ((((size_t)page * 2 + 1) * nkv + head) * page_size + off) * hd;
            *reinterpret_cast<uint4*>(dst + c * 8) = v;
        }
    }
}

RV_EXPORT int rv_rope_cache_write(const void* qkv, const void* bias, int bias_dtype, const int* positions,
                                  const float* cos_t, const float* sin_t, const int* slot_mapping,
                                  void* cache, void* q_out, int n_tokens, int nh, int nkv, int hd,
                                  int page_size, int write_kv, int table_rows, int row_stride,
                                  int dtype, int rot, int in_dtype, cudaStream_t stream) {
    if (n_tokens < 0 || nh <= 0 || nkv <= 0 || hd <= 0 || (hd & 1) || page_size <= 0 || table_rows <= 0)
        return RV_ERR_BAD_SIZE;
    if (rot <= 0 || rot > hd || (rot & 1)) return RV_ERR_BAD_SIZE;
    if ((cos_t == nullptr) != (sin_t == nullptr)) return RV_ERR_BAD_SIZE;
    if (row_stride < (write_kv ? nh + 2 * nkv : nh) * hd) return RV_ERR_BAD_SIZE;
    if (n_tokens == 0) return RV_OK;
    if (in_dtype != dtype) {
        // a float32 product, rotated and stored as bfloat16: the values are rounded once
        if (in_dtype != RV_DTYPE_F32 || dtype != RV_DTYPE_BF16) return RV_ERR_BAD_DTYPE;
        const dim3 grid(n_tokens, write_kv ? nh + 2 * nkv : nh);
        const int threads = hd / 2 >= 128 ? 128 : (hd / 2 >= 64 ? 64 : 32);
        RV_LAUNCH_ST = rv_launch(rope_cache_write_kernel<__nv_bfloat16, float>, dim3(grid), dim3(threads), 0, stream,
            (const float*)qkv, bias, bias_dtype, positions, cos_t, sin_t, slot_mapping, (__nv_bfloat16*)cache,
            (__nv_bfloat16*)q_out, nh, nkv, hd, page_size, write_kv, table_rows, row_stride, rot);
        return rv_launch_status();
    }
    if (dtype == RV_DTYPE_BF16 && rot == hd && hd % 16 == 0 && row_stride % 8 == 0 &&
        (reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(cache)) % 16 == 0) {
        const int items = (write_kv ? nh + nkv : nh) * (hd / 16);
        int threads = 32;
        while (threads < 256 && threads < items) threads <<= 1;
        RV_LAUNCH_ST = rv_launch(rope_cache_write_bf16_vec_kernel, dim3(n_tokens), dim3(threads), 0, stream, 
            (const __nv_bfloat16*)qkv, bias, bias_dtype, positions, cos_t, sin_t, slot_mapping, (__nv_bfloat16*)cache,
            (__nv_bfloat16*)q_out, nh, nkv, hd, page_size, write_kv, table_rows, row_stride);
        return rv_launch_status();
    }
    const dim3 grid(n_tokens, write_kv ? nh + 2 * nkv : nh);
    const int threads = hd / 2 >= 128 ? 128 : (hd / 2 >= 64 ? 64 : 32);
    if (dtype == RV_DTYPE_F32)
        RV_LAUNCH_ST = rv_launch(rope_cache_write_kernel<float>, dim3(grid), dim3(threads), 0, stream, 
            (const float*)qkv, bias, bias_dtype, positions, cos_t, sin_t, slot_mapping, (float*)cache,
            (float*)q_out, nh, nkv, hd, page_size, write_kv, table_rows, row_stride, rot);
    else if (dtype == RV_DTYPE_BF16)
        RV_LAUNCH_ST = rv_launch(rope_cache_write_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream, 
            (const __nv_bfloat16*)qkv, bias, bias_dtype, positions, cos_t, sin_t, slot_mapping,
            (__nv_bfloat16*)cache, (__nv_bfloat16*)q_out, nh, nkv, hd, page_size, write_kv, table_rows, row_stride, rot);
    else
        return RV_ERR_BAD_DTYPE;
    return rv_launch_status();
}

// ------------------------------------------------------------------ SiLU(gate) * up
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t row = idx / inter;
        const int col = (int)(idx - row * inter);
        const float g = rv_to_float(gate_up[row * 2 * inter + col]);
        const float u = rv_to_float(gate_up[row * 2 * inter + inter + col]);
        out[idx] = rv_from_float<T>(g / (1.0f + expf(-g)) * u);
    }
}

// bfloat16 with inter a multiple of 8: 16-byte loads of gate and up, one 16-byte store.
__global__ void silu_mul_bf16_vec_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                         int inter, size_t total_vec) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int vec_per_row = inter >> 3;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_vec; idx += stride) {
        const size_t row = idx / vec_per_row;
        const int c = (int)(idx - row * vec_per_row);
        const uint4 g = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + c * 8);
        const uint4 u = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + inter + c * 8);
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
        const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&u);
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 gf = __bfloat1622float2(gh[j]);
            const float2 uf = __bfloat1622float2(uh[j]);
            oh[j] = __floats2bfloat162_rn(gf.x / (1.0f + expf(-gf.x)) * uf.x, gf.y / (1.0f + expf(-gf.y)) * uf.y);
        }
        *reinterpret_cast<uint4*>(out + row * inter + c * 8) = o;
    }
}

RV_EXPORT int rv_silu_mul(const void* gate_up, void* out, int n_rows, int inter, int dtype, cudaStream_t stream) {
    if (n_rows < 0 || inter <= 0) return RV_ERR_BAD_SIZE;
    if (n_rows == 0) return RV_OK;
    const size_t total = (size_t)n_rows * inter;
    const int threads = 256;
    if (dtype == RV_DTYPE_BF16 && inter % 8 == 0 &&
        (reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) % 16 == 0) {
        const size_t total_vec = total / 8;
        size_t vb = (total_vec + threads - 1) / threads;
        if (vb > (size_t)rv_sm_count() * 32) vb = (size_t)rv_sm_count() * 32;
        RV_LAUNCH_ST = rv_launch(silu_mul_bf16_vec_kernel, dim3((int)vb), dim3(threads), 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out,
                                                                 inter, total_vec);
        return rv_launch_status();
    }
    size_t blocks = (total + threads - 1) / threads;
    if (blocks > (size_t)rv_sm_count() * 16) blocks = (size_t)rv_sm_count() * 16;
    if (dtype == RV_DTYPE_F32)
        RV_LAUNCH_ST = rv_launch(silu_mul_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, inter, total);
    else if (dtype == RV_DTYPE_BF16)
        RV_LAUNCH_ST = rv_launch(silu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
    else
        return RV_ERR_BAD_DTYPE;
    return rv_launch_status();
}

// ------------------------------------------------------------------ random normal fill
// out[i] = mean + std * z_i with z from a counter-based generator: element i is word (i mod 4) of
// Philox-4x32-10 at counter (i / 4, stream) under the key `seed`, two words turned into two
// normals by Box-Muller; so a tensor's values depend on (seed, stream, i) only, not on the launch.
// The reference fills its benchmark weights on the host (v3/crates/rvllm-bench); here the
// random-weights mode of the engine fills them where they live.
template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, long long n, float mean, float std, unsigned long long seed,
                                   unsigned long long stream) {
    const long long quads = (n + 3) / 4;
    for (long long qd = (long long)blockIdx.x * blockDim.x + threadIdx.x; qd < quads; qd += (long long)gridDim.x * blockDim.x) {
        uint32_t c[4] = {(uint32_t)(qd & 0xffffffffll), (uint32_t)((unsigned long long)qd >> 32),
                         (uint32_t)(stream & 0xffffffffull), (uint32_t)(stream >> 32)};
        philox4x32_10(c, (uint32_t)(seed & 0xffffffffull), (uint32_t)(seed >> 32));
        float z[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float u1 = ((float)(c[2 * h] >> 8) + 0.5f) * (1.0f / 16777216.0f);      // (0, 1)
            const float u2 = (float)(c[2 * h + 1] >> 8) * (1.0f / 16777216.0f);           // [0, 1)
            const float r = sqrtf(-2.0f * logf(u1));
            float sn, cs;
            sincospif(2.0f * u2, &sn, &cs);
            z[2 * h] = r * cs;
            z[2 * h + 1] = r * sn;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const long long i = qd * 4 + j;
            if (i < n) out[i] = rv_from_float<T>(mean + std * z[j]);
        }
    }
}

RV_EXPORT int rv_fill_normal(void* out, long long n, float mean, float std, unsigned long long seed,
                             unsigned long long stream_id, int dtype, cudaStream_t stream) {
    if (n < 0 || !(std >= 0.f)) return RV_ERR_BAD_SIZE;
    if (n == 0) return RV_OK;
    const int threads = 256;
    long long blocks = ((n + 3) / 4 + threads - 1) / threads;
    if (blocks > (long long)rv_sm_count() * 16) blocks = (long long)rv_sm_count() * 16;
    if (dtype == RV_DTYPE_F32)
        RV_LAUNCH_ST = rv_launch(fill_normal_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, (float*)out, n, mean, std, seed, stream_id);
    else if (dtype == RV_DTYPE_BF16)
        RV_LAUNCH_ST = rv_launch(fill_normal_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream, (__nv_bfloat16*)out, n, mean, std, seed, stream_id);
    else
        return RV_ERR_BAD_DTYPE;
    return rv_launch_status();
}
