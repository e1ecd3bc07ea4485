// True 32-bit linear layer: out[M, N] = x[M, K] . W[N, K]^T (+ bias[N]) (+ residual[M, N]).
// Plain FFMA on the CUDA cores: no tensor-core instruction is used, so no operand is ever
// rounded to TF32.  Every output element is accumulated over K in one fixed order that does
// not depend on M, so a row's result is bitwise the same whatever else is in the batch.
// Any M, N, K.  64x64 tile per block, 4x4 outputs per thread, K in slices of 16.
//
// Shapes of the layer's five products: v3/crates/rvllm-runtime/src/layer_exec.rs:240-266,
// 433-444, 478-488, 511-522 of the reference (which calls cuBLASLt there); bias as a row
// broadcast and the residual as beta = 1 follow cublaslt.rs:335-368.
#include "common.cuh"

#define TM 64
#define TN 64
#define TK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, const void* __restrict__ bias,
                int bias_dtype, const float* __restrict__ residual, float* __restrict__ out,
                int M, int N, int K) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    __shared__ float xs[TK][TM + 1];
    __shared__ float ws[TK][TN + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += TK) {
        // 64 rows x 16 columns of each operand: 1024 elements, 4 per thread
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = threadIdx.x + r * 256;
            const int row = idx >> 4, col = idx & 15;
            const int k = k0 + col;
            xs[col][row] = (m0 + row < M && k < K) ? x[(size_t)(m0 + row) * K + k] : 0.f;
            ws[col][row] = (n0 + row < N && k < K) ? w[(size_t)(n0 + row) * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += rv_load_param(bias, bias_dtype, n);
            if (residual) v += residual[(size_t)m * N + n];
            out[(size_t)m * N + n] = v;
        }
    }
}

RV_EXPORT int rv_gemm_f32(const float* x, const float* w, const void* bias, int bias_dtype,
                          const float* residual, float* out, int M, int N, int K, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0) return RV_ERR_BAD_SIZE;
    if (M == 0) return RV_OK;
    const dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    if (grid.y > 65535) return RV_ERR_BAD_SIZE;
    RV_LAUNCH_ST = rv_launch(gemm_f32_kernel, dim3(grid), dim3(256), 0, stream, x, w, bias, bias_dtype, residual, out, M, N, K);
    return rv_launch_status();
}
