// Shared helpers of the kernel translation units: error channel, launch accounting,
// dtype access and a few warp primitives.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <string>

#include "schedforge_b200.h"

namespace sfb {

// Per-thread message of the last failure (returned by sfb_last_error).
void set_error(const std::string& message);
sfb_status fail(sfb_status status, const std::string& message);
sfb_status cuda_fail(cudaError_t error, const char* what);

// Launch accounting for sfb_launch_count().
void count_launch(int n = 1);

// Device status word written by bounded waits that gave up (see sfb_device_status).
uint32_t* device_status_word();

// ---- programmatic dependent launch ------------------------------------------------------------
// A kernel launched with launch_dependent() may begin (prologue, loads that do not depend on
// the previous kernel) while the previous kernel of the stream is still finishing; it must call
// grid_dependency_wait() before it touches anything the previous kernel reads or writes.  Under
// an ordinary launch both calls are no-ops.
#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <class... Params, class... Args>
inline cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}
#endif

inline sfb_status check_launch(const char* what) {
    count_launch();
    const cudaError_t error = cudaGetLastError();
    return error == cudaSuccess ? SFB_OK : cuda_fail(error, what);
}

#define SFB_REQUIRE(cond, message)                                            \
    do {                                                                      \
        if (!(cond)) return ::sfb::fail(SFB_INVALID_ARGUMENT, (message));     \
    } while (0)

#define SFB_CUDA(call)                                                        \
    do {                                                                      \
        const cudaError_t sfb_error_ = (call);                                \
        if (sfb_error_ != cudaSuccess) return ::sfb::cuda_fail(sfb_error_, #call); \
    } while (0)

#define SFB_TRY(call)                                                         \
    do {                                                                      \
        const sfb_status sfb_status_ = (call);                                \
        if (sfb_status_ != SFB_OK) return sfb_status_;                        \
    } while (0)

inline cudaStream_t as_stream(sfb_stream stream) { return static_cast<cudaStream_t>(stream); }

inline size_t dtype_size(int dtype) { return dtype == SFB_BF16 ? 2 : 4; }

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Number of SMs of the current device (cached).
int sm_count();

}  // namespace sfb
