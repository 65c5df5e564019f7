// Shared by every kernel file: dtype codes, conversions, error returns.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LQ_F32 0
#define LQ_BF16 1

// Error codes returned by the extern "C" launchers (0 = launched).
#define LQ_OK 0
#define LQ_BAD_DTYPE -1
#define LQ_BAD_SIZE -2
#define LQ_NO_DRIVER -3

#define LQ_EXPORT extern "C" __attribute__((visibility("default")))

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

static inline int lq_launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? LQ_OK : (int)e;
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
