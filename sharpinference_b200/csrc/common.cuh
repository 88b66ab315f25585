// Shared helpers of the sm_100a kernel library.
//
// Every kernel file is a translation unit of its own with a C ABI: plain pointers, sizes
// and a cudaStream_t come in, an int status comes back (0 = launched, otherwise a code of
// SharpiStatus).  No file allocates device memory; scratch is passed in by the caller.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdlib.h>
#include <stdint.h>

enum SharpiStatus : int {
    SHARPI_OK = 0,
    SHARPI_BAD_ARGUMENT = 1,     // a size or option the kernel does not take
    SHARPI_LAUNCH_FAILED = 2,    // cudaGetLastError() after the launch was not cudaSuccess
    SHARPI_UNALIGNED = 3,        // a pointer or stride that breaks an alignment rule
};

enum SharpiDtype : int {
    SHARPI_F32 = 0,
    SHARPI_BF16 = 1,
};

#define SHARPI_API extern "C" __attribute__((visibility("default")))

#define SHARPI_CHECK_LAUNCH()                                       \
    do {                                                            \
        cudaError_t err__ = cudaGetLastError();                     \
        if (err__ != cudaSuccess) return SHARPI_LAUNCH_FAILED;      \
    } while (0)

// Programmatic dependent launch.  A kernel launched with SHARPI_LAUNCH_PDL may be started while the kernel
// before it in the stream is still running, so that its launch and set-up overlap that kernel's tail; it
// must call pdl_wait() before it reads or writes anything that an earlier kernel touches (every such kernel
// calls it on every path, before any return, so completion of a kernel implies completion of those before
// it).  What an earlier kernel wrote is read with ordinary loads, never with __ldg: a load that is declared to
// read memory which does not change during the kernel may be moved ahead of the wait by the compiler.
// Launched the plain way, pdl_wait() does nothing.  sharpi_set_programmatic_launch(0) turns the
// attribute off for the launches of this library (every kernel library exports its own switch).
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

static int sharpi_pdl_flag = 1;
static inline int sharpi_pdl_enabled() { return sharpi_pdl_flag; }
SHARPI_API void sharpi_set_programmatic_launch(int on) { sharpi_pdl_flag = on ? 1 : 0; }

#define SHARPI_LAUNCH_PDL(kernel, grid, block, smem, stream, ...)                                  \
    do {                                                                                           \
        cudaLaunchConfig_t cfg__ = {};                                                             \
        cfg__.gridDim = (grid);                                                                    \
        cfg__.blockDim = (block);                                                                  \
        cfg__.dynamicSmemBytes = (smem);                                                           \
        cfg__.stream = (stream);                                                                   \
        cudaLaunchAttribute attr__[1];                                                             \
        attr__[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                         \
        attr__[0].val.programmaticStreamSerializationAllowed = 1;                                  \
        cfg__.attrs = attr__;                                                                      \
        cfg__.numAttrs = sharpi_pdl_enabled() ? 1 : 0;                                             \
        if (cudaLaunchKernelEx(&cfg__, kernel, __VA_ARGS__) != cudaSuccess) return SHARPI_LAUNCH_FAILED; \
    } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads.  `scratch` holds 32 floats of shared memory.
// Every thread receives the total.  The order of the additions is fixed by the block
// size alone, so a row gives the same sum whatever else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = (lane < nwarps) ? scratch[lane] : 0.0f;
    total = warp_sum(total);
    return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = (lane < nwarps) ? scratch[lane] : -INFINITY;
    total = warp_max(total);
    return total;
}

// How much of the past a query at position `pos` may see (the lowest visible position;
// the highest is `pos` itself).  The same three rules name the cache manager's groups.
enum SharpiMask : int {
    SHARPI_MASK_FULL = 0,    // every earlier position
    SHARPI_MASK_CHUNK = 1,   // positions of the same chunk of `span` positions
    SHARPI_MASK_WINDOW = 2,  // the last `span` positions, the query's own included
};

__host__ __device__ __forceinline__ int visible_lo(int pos, int mask_kind, int span) {
    if (mask_kind == SHARPI_MASK_CHUNK) return (pos / span) * span;
    if (mask_kind == SHARPI_MASK_WINDOW) return pos - span + 1 > 0 ? pos - span + 1 : 0;
    return 0;
}
