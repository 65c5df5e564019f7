// Shared by every kernel file: dtype codes, conversions, error returns.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

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

// ------------------------------------------------------------------ programmatic dependent launch
// Kernels of a step follow one another on one stream.  Launched with launch_pdl, a kernel's
// blocks may be scheduled while the kernel before it is still draining; they run up to
// pdl_wait(), which returns once that kernel has completed and its writes are visible.  What a
// block does before pdl_wait() must not read anything an earlier kernel of the step writes, and
// must write nothing: index arithmetic, and prefetching of weights, which no kernel writes.
// pdl_launch_dependents() lets the kernel after this one be scheduled as early as possible.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline int launch_kernel(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    // LQ_PDL=0 in the environment launches every kernel strictly after the one before it.
    static const bool enabled = [] { const char* v = getenv("LQ_PDL"); return !(v && v[0] == '0'); }();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (enabled && early) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    return e == cudaSuccess ? LQ_OK : (int)e;
}

// A kernel whose blocks may be scheduled before the kernel ahead of it has finished.
template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    return launch_kernel(true, kernel, grid, block, smem, stream, args...);
}
// A kernel that starts only when the kernel ahead of it has finished: for kernels whose blocks
// fill an SM (their waiting blocks would keep the blocks of the kernel ahead off that SM).
template <typename... KArgs, typename... Args>
static inline int launch_after(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               Args... args) {
    return launch_kernel(false, kernel, grid, block, smem, stream, args...);
}
