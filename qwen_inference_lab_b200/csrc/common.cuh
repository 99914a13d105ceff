// Shared helpers of the sm_100a kernels: dtype codes, conversions, reductions and
// the error convention of the exported C entry points.
//
// Every entry point is `extern "C" int qil_<name>(..., cudaStream_t stream)`.
// It returns 0 when the launch was queued, a positive cudaError_t when the launch
// failed, and a negative code when the arguments were refused (the reason is then
// available from qil_last_error()).  Nothing here allocates or synchronises.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#define QIL_F32 0
#define QIL_BF16 1

typedef __nv_bfloat16 bf16;

// One translation unit of every library expands QIL_ERROR_STORAGE; the others
// only see the declaration.
extern thread_local char qil_error_text[512];
#define QIL_ERROR_STORAGE                                                \
    thread_local char qil_error_text[512] = "";                          \
    extern "C" const char* qil_last_error() { return qil_error_text; }

#define QIL_REFUSE(...)                                                  \
    do {                                                                 \
        snprintf(qil_error_text, sizeof(qil_error_text), __VA_ARGS__);   \
        return -1;                                                       \
    } while (0)

#define QIL_CHECK_LAUNCH()                                               \
    do {                                                                 \
        cudaError_t qil_e = cudaGetLastError();                          \
        if (qil_e != cudaSuccess) {                                      \
            snprintf(qil_error_text, sizeof(qil_error_text), "%s",       \
                     cudaGetErrorString(qil_e));                         \
            return (int)qil_e;                                           \
        }                                                                \
        return 0;                                                        \
    } while (0)

// Programmatic dependent launch.  A kernel launched through qil_launch_chained may begin while the
// kernel before it on the stream is still finishing: everything it does before qil_wait_for_producer()
// (fetching weights, which no kernel writes) overlaps that tail; after the wait, all memory the
// earlier kernels wrote is visible.  qil_release_consumer() lets the kernel after this one start as
// soon as every block of this one is past it.  Launched the ordinary way both are no-ops.
__device__ __forceinline__ void qil_wait_for_producer() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void qil_release_consumer() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

#include <stdlib.h>
static inline bool qil_chaining_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* e = getenv("QIL_CHAINED_LAUNCH");
        enabled = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return enabled == 1;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t qil_launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                             cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = qil_chaining_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Round a float to the storage type and back: the value the reference would hold
// after `.to(dtype)`.
template <typename T> __device__ __forceinline__ float round_to(float v) {
    return to_f32<T>(from_f32<T>(v));
}

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

// Block-wide sum with a fixed tree (deterministic for a given block size).
// `scratch` must hold 32 floats.  All threads receive the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = (lane < warps) ? scratch[lane] : 0.f;
    total = warp_sum(total);
    return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = (lane < warps) ? scratch[lane] : -INFINITY;
    total = warp_max(total);
    return total;
}

// Dispatch on (activation dtype, weight dtype) codes.
#define QIL_DISPATCH_2(ACT, WT, ...)                                           \
    do {                                                                       \
        if ((ACT) == QIL_F32 && (WT) == QIL_F32) { typedef float T; typedef float W; __VA_ARGS__; }      \
        else if ((ACT) == QIL_BF16 && (WT) == QIL_BF16) { typedef bf16 T; typedef bf16 W; __VA_ARGS__; } \
        else if ((ACT) == QIL_BF16 && (WT) == QIL_F32) { typedef bf16 T; typedef float W; __VA_ARGS__; } \
        else if ((ACT) == QIL_F32 && (WT) == QIL_BF16) { typedef float T; typedef bf16 W; __VA_ARGS__; } \
        else QIL_REFUSE("unknown dtype codes %d/%d", (int)(ACT), (int)(WT));   \
    } while (0)

#define QIL_DISPATCH_1(ACT, ...)                                               \
    do {                                                                       \
        if ((ACT) == QIL_F32) { typedef float T; __VA_ARGS__; }                \
        else if ((ACT) == QIL_BF16) { typedef bf16 T; __VA_ARGS__; }           \
        else QIL_REFUSE("unknown dtype code %d", (int)(ACT));                  \
    } while (0)
