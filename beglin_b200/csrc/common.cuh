// Shared helpers of the sm_100a kernels: element types, loads and stores that convert to and
// from float, warp and block reductions, and the status word in which a kernel records a bad
// index instead of touching memory it does not own.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define BG_DTYPE_F32 0
#define BG_DTYPE_BF16 1

// Return codes of the extern "C" entry points: 0 is success, a positive value is a cudaError_t,
// a negative one says which argument was refused.
#define BG_OK 0
#define BG_ERR_DTYPE (-1)
#define BG_ERR_SHAPE (-2)
#define BG_ERR_ALIGN (-3)
#define BG_ERR_UNSUPPORTED (-4)

// Bits of the device status word.
#define BG_STATUS_BAD_TOKEN 1u      // a token id outside [0, vocab)
#define BG_STATUS_BAD_PAGE 2u       // a block-table entry outside [0, num_pages)
#define BG_STATUS_TIMEOUT 4u        // a bounded wait ran out

#define BG_LAUNCH_CHECK() \
    do { cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) return (int)e_; } while (0)

namespace bg {

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

}  // namespace bg

// Dispatch on a runtime dtype code to a template argument.
#define BG_DISPATCH_DTYPE(code, T, ...)                                   \
    do {                                                                  \
        if ((code) == BG_DTYPE_F32) { using T = float; __VA_ARGS__; }     \
        else if ((code) == BG_DTYPE_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else return BG_ERR_DTYPE;                                         \
    } while (0)
