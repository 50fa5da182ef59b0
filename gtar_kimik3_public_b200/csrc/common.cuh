// Shared helpers of the sm_100a kernel library: status reporting, type conversion, warp and
// block reductions with a fixed order (the same inputs always reduce in the same order, so a
// row's result never depends on what else is in the launch).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define GK_EXPORT extern "C" __attribute__((visibility("default")))

// Element type codes used across the C interface.
enum GkDtype : int { GK_F32 = 0, GK_BF16 = 1 };

// Status codes returned by every entry point; 0 is success.
enum GkStatus : int { GK_OK = 0, GK_BAD_ARGUMENT = 1, GK_CUDA_ERROR = 2, GK_UNSUPPORTED = 3 };

// Records a message that gk_last_error() returns (one per host thread).
int gk_fail(int status, const char* fmt, ...);

#define GK_REQUIRE(cond, ...)                                \
    do {                                                     \
        if (!(cond)) return gk_fail(GK_BAD_ARGUMENT, __VA_ARGS__); \
    } while (0)

#define GK_CHECK_LAUNCH(name)                                                           \
    do {                                                                                \
        cudaError_t gk_err__ = cudaGetLastError();                                      \
        if (gk_err__ != cudaSuccess)                                                    \
            return gk_fail(GK_CUDA_ERROR, "%s: launch failed: %s", name, cudaGetErrorString(gk_err__)); \
    } while (0)

// Programmatic dependent launch.  A kernel launched with the attribute may start while the kernel
// before it in the stream still runs; it must call pdl_wait() before it touches anything that
// kernel writes (or overwrites anything it reads).  Without the attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

extern int g_gk_pdl;  // set through gk_set_pdl(): launch kernels with programmatic stream serialization
void gk_prepare_kernel(const void* kernel);  // once per kernel: its preferred L1 / shared-memory split

// Launches `kernel` on `stream`, with the programmatic-dependent-launch attribute when it is switched
// on, and as thread-block clusters of `cluster` blocks when that is more than one block.
template <typename... KArgs, typename... Args>
inline cudaError_t gk_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     dim3 cluster, Args... args) {
    gk_prepare_kernel(reinterpret_cast<const void*>(kernel));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (g_gk_pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x;
        attr[n].val.clusterDim.y = cluster.y;
        attr[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    cfg.attrs = n ? attr : nullptr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t gk_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    return gk_launch_cluster(kernel, grid, block, smem, stream, dim3(1, 1, 1), args...);
}

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ float from_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Dispatch on a dtype code: binds `T` in the body.
#define GK_DISPATCH_DTYPE(code, T, ...)                  \
    if ((code) == GK_F32) {                              \
        using T = float;                                 \
        __VA_ARGS__                                      \
    } else {                                             \
        using T = __nv_bfloat16;                         \
        __VA_ARGS__                                      \
    }

#define GK_VALID_DTYPE(code) ((code) == GK_F32 || (code) == GK_BF16)
