// shared by the kernels of libb200mixers.so: type conversion, warp reductions, dtype dispatch
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "b200_mixers.h"

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
// log(sigmoid(z)) without cancellation on either side
__device__ __forceinline__ float log_sigmoid_f(float z) { return z >= 0.0f ? -log1pf(expf(-z)) : z - log1pf(expf(z)); }

#define MIXERS_DISPATCH(dtype, ...)                                                              \
    do {                                                                                         \
        if ((dtype) == 0) { using T = float; __VA_ARGS__; }                                      \
        else if ((dtype) == 1) { using T = __nv_bfloat16; __VA_ARGS__; }                         \
        else if ((dtype) == 2) { using T = __half; __VA_ARGS__; }                                \
        else return (int)cudaErrorInvalidValue;                                                  \
    } while (0)

static inline int mixers_status() { return (int)cudaGetLastError(); }
