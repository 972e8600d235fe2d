// Shared helpers for the hand-written sm_100a kernels: element types, warp
// reductions, the C ABI's error reporting. No PyTorch headers: the library is
// plain CUDA behind extern "C" launchers, loaded with ctypes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define DD_API extern "C" __attribute__((visibility("default")))

enum DdDtype { DD_F32 = 0, DD_BF16 = 1 };
enum DdAct { DD_ACT_NONE = 0, DD_ACT_GELU_NEW = 1, DD_ACT_GELU_ERF = 2 };

// Records a message for dd_last_error() and returns a non-zero code.
int dd_fail(const char* fmt, ...);
// Returns 0 if the last launch was accepted, else records the CUDA error.
int dd_check_launch(const char* what);

template <typename T> struct DdType;
template <> struct DdType<float> { static constexpr int id = DD_F32; };
template <> struct DdType<__nv_bfloat16> { static constexpr int id = DD_BF16; };

__device__ __forceinline__ float dd_to_f32(float v) { return v; }
__device__ __forceinline__ float dd_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T dd_from_f32(float v);
template <> __device__ __forceinline__ float dd_from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 dd_from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float dd_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float dd_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// gelu_new(u) = 0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3))); gelu(u) = 0.5 u (1 + erf(u / sqrt 2)).
__device__ __forceinline__ float dd_activation(float u, int act) {
    if (act == DD_ACT_GELU_NEW) {
        const float c = 0.7978845608028654f;
        return 0.5f * u * (1.0f + tanhf(c * (u + 0.044715f * u * u * u)));
    }
    if (act == DD_ACT_GELU_ERF) return 0.5f * u * (1.0f + erff(u * 0.7071067811865476f));
    return u;
}

static inline int dd_ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Programmatic dependent launch. Every kernel of this library is launched so that it may start
// while the kernel before it on the stream is still running: it does whatever does not depend
// on earlier kernels (barrier set-up, TMEM allocation, prefetching weights), lets its own
// successor start early (dd_launch_dependents) and then waits for the kernel before it to have
// finished and flushed its writes (dd_grid_wait) before it reads or writes anything else in
// global memory. Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void dd_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dd_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

extern int dd_pdl_enabled;      // errors.cu; switched by dd_set_pdl()

template <typename... KArgs, typename... Args>
static inline cudaError_t dd_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = dd_pdl_enabled ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}
