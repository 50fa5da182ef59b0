// Library-wide pieces of the C interface: the per-thread error message and a version probe.

#include <stdarg.h>
#include <stdio.h>

#include <mutex>
#include <unordered_set>

#include "common.cuh"

static thread_local char g_last_error[512] = "";

int gk_fail(int status, const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, args);
    va_end(args);
    return status;
}

int g_gk_pdl = 0;

// Every kernel asks for the largest shared-memory share of the SM's L1/shared-memory array.  An SM changes
// that split only when it is idle, so kernels that prefer different splits cannot be resident side by side,
// and a kernel launched early (programmatic dependent launch) would wait for the SMs to drain instead of
// fetching its weights next to the kernel in front of it.
void gk_prepare_kernel(const void* kernel) {
    static std::mutex lock;
    static std::unordered_set<const void*> seen;
    std::lock_guard<std::mutex> guard(lock);
    if (seen.insert(kernel).second)
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

// Switches programmatic dependent launch on (1) or off (0) for every later kernel launch of the
// library; returns the previous setting.
GK_EXPORT int gk_set_pdl(int on) {
    const int before = g_gk_pdl;
    g_gk_pdl = on ? 1 : 0;
    return before;
}

GK_EXPORT const char* gk_last_error() { return g_last_error; }

// Interface revision: the Python side refuses a library built from other sources.
GK_EXPORT int gk_interface_version() { return 1; }

// Compute capability of the current device as major * 10 + minor, or a negative CUDA error.
GK_EXPORT int gk_device_capability() {
    int device = 0, major = 0, minor = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
    if (err != cudaSuccess) return -(int)err;
    return major * 10 + minor;
}
