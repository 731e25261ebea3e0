// C entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference implementation.
//
// Who needs it: code that runs where cudaMalloc / cudaFree are off limits - inside a
// region that is being captured or replayed by a framework that forbids allocation, in a
// real-time or latency-critical loop where the implicit device synchronisation of an
// allocation is unacceptable, or in a host program that hands this library a fixed memory
// budget up front and has no allocator to lend it.  The regular `chol_inverse` path asks
// its caller for a scratch buffer of batch * r * r floats; such callers cannot provide one.
//
// dion_chol_inverse_noalloc does the same computation as dion::chol_inverse_launch (the
// Cholesky factor inverse Z of every Gram matrix G, see kernels.h) but keeps the scratch in
// a fixed array that is part of the library image: kDionNoAllocScratchFloats floats, held by
// every GPU that loads the library until the process exits.  It calls no cudaMalloc,
// cudaFree or allocating library routine.
//
//   * Inputs and outputs (G, Z, info) are still the caller's device buffers.
//   * batch * r * r must not exceed kDionNoAllocScratchFloats and r must not exceed the
//     largest rank the kernel supports; otherwise nothing is launched, a non-zero code is
//     returned and dion_noalloc_last_error() describes the problem.
//   * The first call on a device looks up the device address of the scratch array (with
//     that device current).  Make that first call before starting any stream capture.
//   * All calls share the one scratch array, which keeps whatever the previous call left in
//     it; every call overwrites the part it uses before reading it.  Calls that can overlap
//     on the GPU (different streams, or different host threads) race on it: serialise them.
//
// Returns 0 on success, 1 for a rejected argument, 2 for a CUDA error.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch array, in floats (8 MiB).
#define kDionNoAllocScratchFloats (2 * 1024 * 1024)

int dion_chol_inverse_noalloc(const float* G, float* Z, int* info, int batch, int r, long long ldg,
                              long long g_batch_stride, float pivot_floor, cudaStream_t stream);

// Message for the last non-zero return value on the calling thread ("" if none).
const char* dion_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
