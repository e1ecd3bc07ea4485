// Weight-streaming linear layer for few rows (decode): out[M, N] = x[M, K] . W[N, K]^T
// (+ bias) (+ residual), or with GATED: out[M, N/2] = silu(g) * u for g = rows [0, N/2) and
// u = rows [N/2, N) of W.  bfloat16 in, float accumulate, bfloat16 or float out.  M <= 64.
//
// Every weight byte is read from HBM exactly once, with 16-byte loads that go straight into
// tensor-core operand registers: the weights are the A operand of mma.sync m16n8k16 (16 output
// features x 16 k), the activations the B operand (16 k x 8 batch rows).  A lane loads 8
// consecutive k of two weight rows; because a dot product does not care in which order k is
// summed, the same k permutation is applied to the activations and no shuffle through shared
// memory is needed for the weights.  The activations of the batch sit in shared memory (staged
// in chunks of K).  A CTA owns NT tiles of 16 output features; its 8 warps split K and their
// partial sums are added through shared memory in a fixed order, so a row's result does not
// depend on what else is in the batch.
//
// Shapes served: the five products of a layer and the LM head at decode time
// (v3/crates/rvllm-runtime/src/layer_exec.rs:240-266,433-444,478-488,511-522 and
// bring_up.rs:648-658 of the reference, which calls cuBLASLt; its SiLU kernel layout
// kernels/fused_silu_fp8_quant.cu:52-56 is the [gate | up] pairing used by GATED).
#include "common.cuh"

#define SK_WARPS 8
#define SK_THREADS (SK_WARPS * 32)
#define X_PAD 32   // bf16 elements (64 bytes) of padding per activation row in shared memory

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct SkinnyParams {
    const __nv_bfloat16* x;       // [M, K]
    const __nv_bfloat16* w;       // [N, K]
    const void* bias;             // [N] or null
    int bias_dtype;
    const __nv_bfloat16* residual;  // [M, N_out] or null
    void* out;                    // [M, N_out]
    int out_f32;
    int M, N, K;
    int kc;                       // K chunk staged in shared memory (multiple of 32)
};

template <int MT, int NT, bool GATED>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const SkinnyParams p) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int quad = lane >> 2, tq = lane & 3;
    const int xs_stride = p.kc + X_PAD;
    const int half_n = p.N >> 1;
    // first output feature of each of this CTA's tiles
    int n_base[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        if (GATED) {
            const int pair = blockIdx.x * (NT / 2) + (nt >> 1);
            n_base[nt] = pair * 16 + ((nt & 1) ? half_n : 0);
        } else {
            n_base[nt] = (blockIdx.x * NT + nt) * 16;
        }
    }
    const int n_limit = GATED ? half_n : p.N;      // rows of a tile beyond this are not real
    float acc[NT][MT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) { acc[nt][mt][0] = acc[nt][mt][1] = acc[nt][mt][2] = acc[nt][mt][3] = 0.f; }

    // weight row pointers of this lane: rows quad and quad + 8 of each tile
    const __nv_bfloat16* wrow[NT][2];
    bool wok[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int local = quad + 8 * h;
            const int base = GATED ? (n_base[nt] - ((nt & 1) ? half_n : 0)) : n_base[nt];
            wok[nt][h] = base + local < n_limit;
            wrow[nt][h] = p.w + (size_t)(wok[nt][h] ? n_base[nt] + local : 0) * p.K;
        }

    for (int c0 = 0; c0 < p.K; c0 += p.kc) {
        const int kc = min(p.kc, p.K - c0);            // multiple of 8
        const int kc32 = (kc + 31) & ~31;
        __syncthreads();
        // stage x[:, c0 : c0 + kc] (rows >= M and columns >= kc are zero)
        const int chunks = kc32 >> 3;
        for (int idx = tid; idx < MT * 8 * chunks; idx += SK_THREADS) {
            const int m = idx / chunks, c = idx - m * chunks;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (m < p.M && c * 8 < kc) v = *reinterpret_cast<const uint4*>(p.x + (size_t)m * p.K + c0 + c * 8);
            *reinterpret_cast<uint4*>(xs + (size_t)m * xs_stride + c * 8) = v;
        }
        __syncthreads();
        const int nsteps = kc32 >> 5;
#pragma unroll 2
        for (int s = warp; s < nsteps; s += SK_WARPS) {
            const int k = s * 32 + tq * 8;               // within the chunk
            const bool kok = k < kc;
            uint4 a[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    a[nt][h] = (kok && wok[nt][h]) ? __ldcs(reinterpret_cast<const uint4*>(wrow[nt][h] + c0 + k))
                                                   : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const uint4 b = *reinterpret_cast<const uint4*>(xs + (size_t)(mt * 8 + quad) * xs_stride + k);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mma_bf16_16816(acc[nt][mt], a[nt][0].x, a[nt][1].x, a[nt][0].y, a[nt][1].y, b.x, b.y);
                    mma_bf16_16816(acc[nt][mt], a[nt][0].z, a[nt][1].z, a[nt][0].w, a[nt][1].w, b.z, b.w);
                }
            }
        }
    }

    // add the 8 warps' partial sums in warp order
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem_raw);       // [SK_WARPS][NT * 16][MT * 8]
    constexpr int TILE_ELEMS = NT * 16 * MT * 8;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float* dst = red + (size_t)warp * TILE_ELEMS + (nt * 16 + quad) * (MT * 8) + mt * 8 + tq * 2;
            dst[0] = acc[nt][mt][0]; dst[1] = acc[nt][mt][1];
            dst[8 * MT * 8] = acc[nt][mt][2]; dst[8 * MT * 8 + 1] = acc[nt][mt][3];
        }
    __syncthreads();
    if (GATED) {
        constexpr int PAIRS = NT / 2;
        for (int idx = tid; idx < PAIRS * 16 * MT * 8; idx += SK_THREADS) {
            const int m = idx % (MT * 8);
            const int rest = idx / (MT * 8);
            const int local = rest % 16, pair = rest / 16;
            float g = 0.f, u = 0.f;
#pragma unroll
            for (int w = 0; w < SK_WARPS; ++w) {
                g += red[(size_t)w * TILE_ELEMS + ((2 * pair) * 16 + local) * (MT * 8) + m];
                u += red[(size_t)w * TILE_ELEMS + ((2 * pair + 1) * 16 + local) * (MT * 8) + m];
            }
            const int n = n_base[0] + pair * 16 + local;      // tiles of a CTA are consecutive pairs
            if (m < p.M && n < half_n) {
                const float v = g / (1.0f + expf(-g)) * u;
                if (p.out_f32) ((float*)p.out)[(size_t)m * half_n + n] = v;
                else ((__nv_bfloat16*)p.out)[(size_t)m * half_n + n] = __float2bfloat16_rn(v);
            }
        }
    } else {
        for (int idx = tid; idx < TILE_ELEMS; idx += SK_THREADS) {
            const int m = idx % (MT * 8);
            const int row = idx / (MT * 8);                 // nt * 16 + local
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < SK_WARPS; ++w) v += red[(size_t)w * TILE_ELEMS + idx];
            const int n = n_base[0] + row;                   // tiles of a CTA are consecutive
            if (m < p.M && n < p.N) {
                if (p.bias) v += rv_load_param(p.bias, p.bias_dtype, n);
                if (p.residual) v += __bfloat162float(p.residual[(size_t)m * p.N + n]);
                if (p.out_f32) ((float*)p.out)[(size_t)m * p.N + n] = v;
                else ((__nv_bfloat16*)p.out)[(size_t)m * p.N + n] = __float2bfloat16_rn(v);
            }
        }
    }
}

template <int MT, int NT, bool GATED>
static int launch_skinny(SkinnyParams& p, cudaStream_t stream) {
    // K chunk: as large as fits beside nothing else; shared memory is reused for the reduction
    const int budget = 160 * 1024;
    // a multiple of 32 * SK_WARPS: warp w then owns the k steps congruent to w whatever the chunk
    // size is, so the order of summation does not depend on M
    int kc = (budget / (MT * 8 * 2)) - X_PAD;
    kc &= ~(32 * SK_WARPS - 1);
    const int k32 = (p.K + 32 * SK_WARPS - 1) & ~(32 * SK_WARPS - 1);
    if (kc > k32) kc = k32;
    p.kc = kc;
    const size_t x_bytes = (size_t)MT * 8 * (kc + X_PAD) * 2;
    const size_t red_bytes = (size_t)SK_WARPS * NT * 16 * MT * 8 * 4;
    const size_t smem = x_bytes > red_bytes ? x_bytes : red_bytes;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<MT, NT, GATED>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int rows_per_cta = GATED ? (NT / 2) * 16 : NT * 16;
    const int n_rows = GATED ? p.N / 2 : p.N;
    const int grid = (n_rows + rows_per_cta - 1) / rows_per_cta;
    RV_LAUNCH_ST = rv_launch(gemm_skinny_kernel<MT, NT, GATED>, dim3(grid), dim3(SK_THREADS), smem, stream, p);
    return rv_launch_status();
}

template <int MT>
static int dispatch_nt(SkinnyParams& p, int gated, int nt, cudaStream_t stream) {
    if (gated) return nt >= 4 ? launch_skinny<MT, 4, true>(p, stream) : launch_skinny<MT, 2, true>(p, stream);
    if (nt >= 4) return launch_skinny<MT, 4, false>(p, stream);
    if (nt == 2) return launch_skinny<MT, 2, false>(p, stream);
    return launch_skinny<MT, 1, false>(p, stream);
}

// gated = 1: W rows are [gate | up], the output is silu(gate) * up with N/2 columns (no bias, no
// residual).  tiles_per_cta: 1, 2 or 4 tiles of 16 output features per CTA (0: chosen here so
// that the grid covers the GPU about twice).
RV_EXPORT int rv_gemm_skinny_bf16(const void* x, const void* w, const void* bias, int bias_dtype,
                                  const void* residual, void* out, int out_f32, int M, int N, int K,
                                  int gated, int tiles_per_cta, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0) return RV_ERR_BAD_SIZE;
    if (M > 64) return RV_ERR_UNSUPPORTED;
    if (K % 8) return RV_ERR_UNSUPPORTED;          // weight rows must start on 16-byte boundaries
    if (gated && ((N & 1) || bias || residual)) return RV_ERR_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16) return RV_ERR_ALIGNMENT;
    if (M == 0) return RV_OK;
    SkinnyParams p;
    p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.bias = bias; p.bias_dtype = bias_dtype;
    p.residual = (const __nv_bfloat16*)residual; p.out = out; p.out_f32 = out_f32;
    p.M = M; p.N = N; p.K = K; p.kc = 0;
    const int mt = (M + 7) / 8;
    int nt = tiles_per_cta;
    if (nt <= 0) {
        const int tiles = ((gated ? N / 2 : N) + 15) / 16 * (gated ? 2 : 1);
        nt = tiles >= 4 * 296 ? 4 : (tiles >= 2 * 296 ? 2 : 1);
        if (mt > 4 && nt > 2) nt = 2;                // keep the accumulators in registers
    }
    if (gated && nt < 2) nt = 2;
    if (mt <= 1) return dispatch_nt<1>(p, gated, nt, stream);
    if (mt <= 2) return dispatch_nt<2>(p, gated, nt, stream);
    if (mt <= 4) return dispatch_nt<4>(p, gated, nt, stream);
    return dispatch_nt<8>(p, gated, nt, stream);
}
