// Shared helpers of the hand-written sm_100a kernels: dtype-generic loads and stores that
// compute in float, warp and block reductions, and the launch-status convention.
//
// Every exported launcher returns 0 on success or a negative code for sizes it refuses
// (never a wrong result); a CUDA launch error is returned as the positive cudaError_t.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define RV_OK 0
#define RV_ERR_BAD_SIZE (-1)
#define RV_ERR_BAD_DTYPE (-2)
#define RV_ERR_ALIGNMENT (-3)
#define RV_ERR_UNSUPPORTED (-4)

#define RV_DTYPE_F32 0
#define RV_DTYPE_BF16 1

#define RV_EXPORT extern "C" __attribute__((visibility("default")))

// ---- programmatic dependent launch ---------------------------------------------------------
// Kernels of a step run back to back on one stream.  Launched with the programmatic-serialization
// attribute, a kernel may be scheduled while its predecessor is still running: what it does before
// rv_pdl_wait() (set-up, fetching weights, which no kernel of the step writes) overlaps the
// predecessor's tail; everything after rv_pdl_wait() sees the predecessor complete.  Without the
// attribute both calls do nothing.  The switch is per library (rv_set_pdl).
// Two rules for what runs before rv_pdl_wait(): it reads only what no kernel of the step writes
// (weights, the step's metadata), and it writes no global memory at all - a buffer handed out by a
// stream-ordered allocator may still be in use, under another name, by a kernel running ahead.
static int g_rv_pdl = 0;
RV_EXPORT void rv_set_pdl(int on) { g_rv_pdl = on; }

__device__ __forceinline__ void rv_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void rv_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline int rv_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_rv_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    return RV_OK;
}

// The same with the grid's CTAs grouped into clusters of `cluster_x` along x (distributed shared memory).
template <typename... KArgs, typename... Args>
static inline int rv_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    unsigned cluster_x, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_rv_pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    return RV_OK;
}

// ---- per-device set-up -----------------------------------------------------------------------
// cudaFuncSetAttribute and the number of SMs belong to a device, not to the process: a library
// used on a second GPU has to set its kernels up there as well.  `RvPerDevice` remembers, per
// device ordinal, that a one-time set-up ran (two host threads that meet in a first call both
// run it and store the same value).
#define RV_MAX_DEVICES 64
struct RvPerDevice { bool done[RV_MAX_DEVICES]; };

static inline int rv_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= RV_MAX_DEVICES) return -1;
    return dev;
}

// Raises the dynamic shared memory limit of `kernel` to `bytes` once per device.
template <typename K>
static inline int rv_configure_smem(RvPerDevice& once, K kernel, int bytes) {
    const int dev = rv_current_device();
    if (dev >= 0 && once.done[dev]) return RV_OK;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    if (dev >= 0) once.done[dev] = true;
    return RV_OK;
}

// The number of SMs of the current device (asked once per device).
static inline int rv_sm_count() {
    static int sms[RV_MAX_DEVICES];
    const int dev = rv_current_device();
    if (dev >= 0 && sms[dev] > 0) return sms[dev];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev < 0 ? 0 : dev) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return 148;
    }
    if (dev >= 0) sms[dev] = n;
    return n;
}

// the status of the most recent rv_launch of this thread (launchers write RV_LAUNCH_ST = rv_launch(...))
static thread_local int rv_launch_st = 0;
#define RV_LAUNCH_ST rv_launch_st

static inline int rv_launch_status() {
    const int s = rv_launch_st;
    rv_launch_st = 0;
    if (s != RV_OK) return s;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? RV_OK : (int)e;
}

// Philox-4x32-10 (Salmon et al., 2011): counter c, key (k0, k1) -> four random words in c.
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

__device__ __forceinline__ float rv_to_float(float v) { return v; }
__device__ __forceinline__ float rv_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T rv_from_float(float v);
template <> __device__ __forceinline__ float rv_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 rv_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// A vector parameter (norm weight, bias) may be stored in either type, whatever the
// activations are: a tensor that the checkpoint holds in 32 bits stays in 32 bits.
__device__ __forceinline__ float rv_load_param(const void* p, int dtype, int i) {
    return dtype == RV_DTYPE_F32 ? ((const float*)p)[i]
                                 : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

__device__ __forceinline__ float rv_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float rv_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float rv_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = rv_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = rv_warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float rv_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = rv_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = rv_warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
