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

// ---- whole lines to memory.  A thread of the output stage owns one row of the tile, so a store instruction of
// its warp touches 32 different lines with 16 bytes each, and the memory pipeline takes such requests at about
// one in two cycles: the stores of a 128 x 256 tile then cost as much as its multiplications (measured: 650 to
// 1,100 cycles for sixteen columns, against 28 for reading them out of tensor memory).  Shared memory is no
// way round it, for the MMAs need its bandwidth.  So four lanes with four consecutive rows swap, by shuffles,
// the four 32-byte pieces of 128 bytes of their rows: lane 4j + m ends up with piece m of the rows 4j .. 4j + 3,
// and each of four 32-byte stores of the warp fills eight whole lines.
__device__ __forceinline__ void pack8(const float* v, uint32_t* r) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        r[i] = *reinterpret_cast<uint32_t*>(&h);
    }
}

// in: r[P m .. P m + P - 1] = piece m of this lane's row;  out: r[P i .. P i + P - 1] = piece (lane % 4) of row (lane - lane % 4) + i
template <typename T, int P>
__device__ __forceinline__ void swap_pieces(T* r, int lane) {
#pragma unroll
    for (int bit = 0; bit < 2; ++bit) {
        const int step = 1 << bit;           // partner lane ^ step; slots s and s + step with (s & step) == 0
        const bool upper = (lane & step) != 0;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            if (s & step) continue;
#pragma unroll
            for (int e = 0; e < P; ++e) {
                T& lo = r[s * P + e];
                T& hi = r[(s + step) * P + e];
                const T got = __shfl_xor_sync(0xffffffffu, upper ? lo : hi, step);
                if (upper) lo = got;
                else hi = got;
            }
        }
    }
}

// 32 bytes of a table that no kernel in flight writes (not volatile: the compiler may issue it early)
__device__ __forceinline__ void load32(const float* src, float (&v)[8]) {
    asm("ld.global.nc.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]) : "l"(src));
}
// 32 bytes that an earlier kernel may have written
__device__ __forceinline__ void load32(const void* src, uint32_t (&v)[8]) {
    asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "l"(src) : "memory");
}
__device__ __forceinline__ void store32(void* dst, const uint32_t* r) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]),
                 "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
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
