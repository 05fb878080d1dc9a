// mhb_gemm_simt_noalloc: the split-K CUDA-core matrix product with its scratch built into the
// library, for callers that must not allocate device memory.
//
// This entry point has no counterpart in KiritoHugh/mini-hisparse; it is an addition of this
// engine's kernel library.
//
// Who needs it.  The split-K product writes one partial matrix per K split and then sums them, so
// it needs nsplit * M * N floats of scratch.  mhb_gemm_simt leaves that buffer to the caller, which
// is fine for the engine (its workspace comes from torch's allocator).  It is not fine for a caller
// that cannot call cudaMalloc at the moment of the product:
//   * code running while a stream is being captured into a CUDA graph (an allocation is refused
//     during capture, and one made before it would have to be planned by someone else);
//   * a serving loop that has handed all free device memory to its KV page pool, so that an
//     allocation may fail or trigger a device-wide synchronisation at an unpredictable moment;
//   * a plug-in that is given device pointers by its host program and is not allowed to own memory.
// For them the scratch is a fixed array inside the library: MHB_NOALLOC_SCRATCH_FLOATS floats
// (8 MiB) of device memory on every GPU that loads the library, held until the process exits.
//
// Contract.
//   * C [M, N] float32 (row stride ldc) = A [M, K] * W [N, K]^T, float32 accumulation; A and W are
//     float32 or bfloat16 (dtype codes 0 / 1), row-major with K contiguous.  Inputs and the output
//     are the caller's; the entry point calls no cudaMalloc, cudaFree or any allocating routine.
//   * nsplit * M * N must not exceed MHB_NOALLOC_SCRATCH_FLOATS; larger products are refused with
//     an error text (mhb_last_error) and nothing is launched.  So are more than 65535 splits and
//     an output row stride shorter than N.  Splits beyond the K range are allowed: they add zeros.
//   * Host threads may call at the same time as far as the address look-up goes (it is locked);
//     the rule on overlapping kernels below holds for them as for streams.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current).  Make that first call before any stream capture begins.
//   * All calls share the one array, and it keeps whatever the last call left in it.  The product
//     never reads an element it has not written in the same call, so nothing has to be cleared;
//     but two calls whose kernels overlap on the GPU (different streams, no ordering between them)
//     race on the array.  Order such calls, or give each its own stream-ordered turn.
// Returns 0, or a negative code with the text in mhb_last_error().
#pragma once
#include <cuda_runtime.h>

#define MHB_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C"
#endif
int mhb_gemm_simt_noalloc(const void* A, int a_dtype, const void* W, int w_dtype, float* C, int M, int N,
                          int K, long long lda, long long ldw, long long ldc, int nsplit,
                          cudaStream_t stream);
