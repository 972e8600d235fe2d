// Error reporting of the C ABI: every launcher returns 0 or records one message.
#include "common.cuh"
#include <stdarg.h>
#include <stdio.h>

static thread_local char g_message[512] = "";

int dd_fail(const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_message, sizeof(g_message), fmt, args);
    va_end(args);
    return 1;
}

int dd_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return dd_fail("%s: %s", what, cudaGetErrorString(e));
    return 0;
}

int dd_pdl_enabled = 1;

// 1 (default): kernels are launched with programmatic stream serialization, so each may start
// its set-up while its predecessor still runs; 0: ordinary stream order. Returns the old value.
DD_API int dd_set_pdl(int enabled) {
    const int old = dd_pdl_enabled;
    dd_pdl_enabled = enabled ? 1 : 0;
    return old;
}

DD_API const char* dd_last_error() { return g_message; }

// Compute capability of the current device as major*10+minor, or a negative CUDA error.
DD_API int dd_device_arch() {
    int dev = 0, major = 0, minor = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    return major * 10 + minor;
}

// One asynchronous copy of `bytes` bytes from pinned host memory to the device, in stream order: the step's
// metadata, without a framework call in between.
DD_API int dd_copy_to_device(void* dst, const void* src, long long bytes, void* stream) {
    if (bytes <= 0) return 0;
    cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream);
    if (e != cudaSuccess) return dd_fail("dd_copy_to_device: %s", cudaGetErrorString(e));
    return 0;
}
