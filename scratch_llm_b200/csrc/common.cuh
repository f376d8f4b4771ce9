// Shared device helpers for the engine's kernels (sm_100a).
//
// Every launcher is an extern "C" function that takes raw device pointers, sizes and the
// CUDA stream to launch on, allocates nothing, and returns a cudaError_t as int (0 = ok).
// Launchers check sizes they cannot handle and return cudaErrorInvalidValue instead of
// computing a wrong result; the Python binding turns any non-zero code into an exception.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SLLM_EXPORT extern "C" __attribute__((visibility("default")))

#define SLLM_LAUNCH_CHECK()                          \
    do {                                             \
        cudaError_t e__ = cudaGetLastError();        \
        if (e__ != cudaSuccess) return (int)e__;     \
    } while (0)

namespace sllm {

// Programmatic dependent launch.  pdl_trigger() lets the next kernel in the stream start to be
// scheduled while this one still runs; it only takes effect if that kernel was launched with
// the programmatic-stream-serialization attribute, and such a kernel must call pdl_wait()
// before it reads or writes anything an earlier kernel may touch (weights, which nothing
// writes, may be read before).  pdl_wait() returns once all earlier kernels have completed
// and their writes are visible; without the launch attribute it returns at once.
// Every kernel here calls pdl_wait() FIRST and pdl_trigger() right after it: a trigger before
// the wait would let the whole chain of later kernels pile up on the SMs, each parked in its
// wait and holding registers and shared memory that the running kernel needs (measured: the
// decode step became 60 % slower).  This way at most one kernel is parked ahead.
__device__ __forceinline__ void pdl_trigger() {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
}

}  // namespace sllm

// Launch with programmatic stream serialization: the kernel may be scheduled while the previous
// kernel of the stream drains, and must call sllm::pdl_wait() before touching that kernel's data.
template <typename... KArgs, typename... Args>
static inline cudaError_t sllm_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                          size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

namespace sllm {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
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

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33
// floats of shared memory.  The order of the additions depends only on blockDim.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace sllm
