// sharpi_sample_rows_no_alloc: token sampling for hosts that may not allocate device memory.
//
// This entry point has no counterpart in pekkah/SharpInference; it is an addition of this library.
//
// Who it is for.  sharpi_sample_rows needs a [rows, vocab] float work area that its caller has to
// provide, which in practice means a device allocation per call or a pool the caller manages.  Some
// hosts of this library can do neither: a C or C++ serving loop that was handed a fixed partition of
// the device's memory at start-up and must not grow it; a plug-in that runs inside another program's
// memory budget, where a cudaMalloc of its own could fail or, because cudaMalloc and cudaFree
// synchronise the device, stall every stream of that program in the middle of a decode step; code
// that runs where the allocator it would normally borrow from (torch's) is not loaded at all.  For
// them the work area lives inside the library: one file-scope __device__ array of
// SHARPI_NO_ALLOC_MAX_FLOATS floats (16 MiB), which every GPU that loads libsampling.so holds until
// the process exits, whether or not this entry point is ever called.
//
// Contract.
//  * Inputs and output are the caller's, exactly as for sharpi_sample_rows (same argument meaning,
//    minus the work area): logits [rows, vocab] float32, per-row temperature, top_k, top_p, min_p and
//    uniform numbers, out [rows] int32; all device pointers; launched on `stream`.
//  * rows * vocab must not exceed SHARPI_NO_ALLOC_MAX_FLOATS; a larger request is refused with
//    SHARPI_NO_ALLOC_TOO_LARGE before anything is launched and `out` is left untouched.
//  * The function calls no cudaMalloc, cudaFree or other allocating routine, of CUDA's or anyone's.
//  * First call on a device: the function looks up the device address of the work area with
//    cudaGetSymbolAddress, with that device current, and remembers it per device.  That first call may
//    make the CUDA runtime load this library's device code, so make it once during start-up, on
//    every device you will use, before any stream capture begins.  Later calls only launch.
//  * All calls share the one work area, and it keeps whatever the previous call left in it.  The
//    kernel overwrites every element it later reads (a row's probabilities are written in full before
//    they are filtered), so nothing needs clearing between calls.  Two calls whose kernels overlap on
//    the GPU (different streams without an ordering between them, or different host threads) race on
//    the work area and produce garbage: order them.
#pragma once

#include <cuda_runtime.h>

#define SHARPI_NO_ALLOC_MAX_FLOATS (4u << 20)   // 4 Mi floats = 16 MiB, e.g. 20 rows of a 202,048-token vocabulary

#define SHARPI_NO_ALLOC_TOO_LARGE 4             // rows * vocab beyond SHARPI_NO_ALLOC_MAX_FLOATS
#define SHARPI_NO_ALLOC_SETUP_FAILED 5          // cudaGetDevice or cudaGetSymbolAddress did not succeed

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default")))
int sharpi_sample_rows_no_alloc(const float* logits, int rows, int vocab, const float* temperature,
                                const int* top_k, const float* top_p, const float* min_p, const float* uniform,
                                int* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
