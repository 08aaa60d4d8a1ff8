// Shared helpers of the kernel sources: element types, conversions, error codes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <utility>

#define CELLM_API extern "C" __attribute__((visibility("default")))

// Element type tags passed from the host.
enum { CELLM_F32 = 0, CELLM_BF16 = 1 };

// Return codes of the C entry points: 0 = launched; a positive value is a
// cudaError_t; a negative value means the entry point refused its arguments.
enum {
    CELLM_OK = 0,
    CELLM_ERR_DTYPE = -1,   // unknown element type tag
    CELLM_ERR_SIZE = -2,    // a size the kernel does not take
    CELLM_ERR_ALIGN = -3,   // a pointer or stride that breaks an alignment rule
    CELLM_ERR_ARG = -4      // a missing or contradictory argument
};

// Bits of the device-side error word that kernels set instead of trapping.
enum {
    CELLM_DEV_BAD_TOKEN = 1,   // token id outside the vocabulary
    CELLM_DEV_BAD_PAGE = 2,    // page id outside the pool
    CELLM_DEV_BAD_SLOT = 4,    // state slot outside the pool
    CELLM_DEV_WAIT_TIMEOUT = 8,// a bounded wait inside a kernel gave up
    CELLM_DEV_BAD_LAYOUT = 16  // shared memory not aligned as the kernel's tiles need
};

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

// Sum over a block in a fixed order (warp trees, then warp 0 over the warps'
// sums), so the result depends only on the values and the block size.
// `scratch` holds at least 32 floats. Every thread gets the sum.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : 0.f;
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

// ---- programmatic dependent launch -----------------------------------------
// Kernels are launched with the attribute that lets the next kernel of the
// stream start while the previous one is still running. Every kernel therefore
// calls pdl_wait() before it reads anything an earlier kernel wrote and before
// it writes anything an earlier kernel may still read; what comes before the
// wait (barrier set-up, tensor-memory allocation, loads of weights) overlaps
// the tail of the previous kernel. pdl_trigger() lets the following kernel
// begin its own preamble.
//
// Some kernels go further and read, before their wait, data that only an
// EARLIER STEP wrote (the convolution's state, keys and values that were in
// the cache before this step). With small grids several kernels can be in
// flight at once, so this is safe only if a step's kernels cannot overlap the
// previous step's. The invariant: the first kernel of every forward pass (the
// embedding) is launched WITHOUT the attribute (cellm_launch_serial), so it
// starts only when everything before it on the stream has finished, and every
// later kernel of the pass waits, directly or through its predecessors, on it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t cellm_launch_with(int overlap, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = overlap;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t cellm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args&&... args) {
    return cellm_launch_with(1, kernel, grid, block, smem, stream, std::forward<Args>(args)...);
}
// The launch of a step's first kernel: it may not begin before the stream's earlier work has finished.
template <typename... KArgs, typename... Args>
inline cudaError_t cellm_launch_serial(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                       Args&&... args) {
    return cellm_launch_with(0, kernel, grid, block, smem, stream, std::forward<Args>(args)...);
}

#define CELLM_RUN(kernel, grid, block, smem, stream, ...)                                   \
    do {                                                                                    \
        cudaError_t e__ = cellm_launch(kernel, dim3(grid), dim3(block), smem, stream, __VA_ARGS__); \
        if (e__ != cudaSuccess) return (int)e__;                                            \
    } while (0)

#define CELLM_RUN_SERIAL(kernel, grid, block, smem, stream, ...)                            \
    do {                                                                                    \
        cudaError_t e__ = cellm_launch_serial(kernel, dim3(grid), dim3(block), smem, stream, __VA_ARGS__); \
        if (e__ != cudaSuccess) return (int)e__;                                            \
    } while (0)

#define CELLM_LAUNCH_CHECK()                         \
    do {                                             \
        cudaError_t e__ = cudaGetLastError();        \
        if (e__ != cudaSuccess) return (int)e__;     \
    } while (0)
