// Shared device helpers for the celeg_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace celeg_b200 {

// Activation/storage element types are chosen at run time by an int code.
enum DType : int { kFloat32 = 0, kBFloat16 = 1 };

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                       // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Programmatic dependent launch. A kernel launched through launch_chained() may start while its
// predecessor in the stream is still running; it must call chain_wait() before it reads anything
// a predecessor wrote and before it writes anything a predecessor may still read (only constant
// data such as weights may be touched earlier). chain_release() lets the successor start
// launching; the successor's chain_wait() still returns only when this whole grid has finished
// and its writes are visible, so releasing early is always safe. It is not always faster: the
// small-batch product releases nothing before its blocks exit (released at its start, or after its main
// loop, a decode step of 74 kernels measured 0.75-0.90 ms instead of 0.70; with the attribute alone it is
// 2 % faster than without).
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;"); }

// Host side: the last error text of this library (thread local).
void set_error(const char* format, ...);
int check_launch(const char* what);
bool chaining_enabled(int kernel_class = 2);
enum ChainClass : int { kChainGemv = 0, kChainNorm = 1, kChainOther = 2 };

// Launch with the programmatic-serialization attribute (when enabled), so that the kernel's
// prologue overlaps the tail of the kernel before it. Works under stream capture as well.
template <typename... KernelArgs, typename... Args>
inline void launch_chained_class(int kernel_class, void (*kernel)(KernelArgs...), dim3 grid, dim3 block,
                                 size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = chaining_enabled(kernel_class) ? 1 : 0;
    config.attrs = attribute;
    config.numAttrs = 1;
    cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

template <typename... KernelArgs, typename... Args>
inline void launch_chained(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                           Args&&... args) {
    launch_chained_class(kChainOther, kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
}

}  // namespace celeg_b200

#define CELEG_API extern "C" __attribute__((visibility("default")))

#define CELEG_REQUIRE(cond, ...)                          \
    do {                                                  \
        if (!(cond)) {                                    \
            ::celeg_b200::set_error(__VA_ARGS__);         \
            return -1;                                    \
        }                                                 \
    } while (0)
