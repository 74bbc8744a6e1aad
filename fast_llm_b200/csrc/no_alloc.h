/* Entry point for callers that cannot allocate device memory.
 *
 * This function has no counterpart in the reference framework; it exists for hosts of this library that are not
 * allowed to call cudaMalloc at the moment they need the result - for example code that runs inside a region where
 * the CUDA allocator is locked down (a memory pool frozen for the duration of a job), or an embedding application
 * that hands this library a fixed budget of device memory up front and forbids any further allocation.  The regular
 * entry point `flb_sumsq` asks such callers for a scratch buffer they have no way to obtain.
 *
 * `flb_sumsq_no_alloc` computes out[0] (+)= sum(x[i]^2) exactly like `flb_sumsq` (same kernels, same deterministic
 * two-stage reduction), but keeps its per-block partial sums in an array that is part of the library image
 * (FLB_NO_ALLOC_SCRATCH_FLOATS floats, 4 KiB, resident on every GPU that loads the library until the process exits).
 * It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 *   x           device pointer, 16-byte aligned, n fp32 values
 *   n           0 <= n <= FLB_NO_ALLOC_MAX_ELEMENTS; larger inputs are rejected with status 4 (FLB_ERR_TOO_LARGE)
 *   out         device pointer to one float; overwritten, or added to when accumulate != 0
 *   stream      stream the work is enqueued on
 *
 * Returns 0 on success, 1 for a misaligned or negative-size input, 2 when a CUDA call failed (see
 * flb_last_cuda_error), 4 when n exceeds the maximum.
 *
 * The first call on each device looks up the device address of the built-in scratch array (cudaGetSymbolAddress, with
 * that device current).  Make that first call outside of any stream capture.  All calls share the one array, which
 * keeps whatever the previous call left in it; every call rewrites all of it before reading, so nothing needs to be
 * cleared, but two calls whose kernels overlap on the GPU (different streams without ordering between them) race on
 * it and give wrong results - order them.
 */
#ifndef FLB_NO_ALLOC_H
#define FLB_NO_ALLOC_H

#include <cuda_runtime.h>

#define FLB_NO_ALLOC_SCRATCH_FLOATS 1024
#define FLB_NO_ALLOC_MAX_ELEMENTS (1ll << 32)

#ifdef __cplusplus
extern "C" {
#endif

int flb_sumsq_no_alloc(const float* x, long long n, float* out, int accumulate, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* FLB_NO_ALLOC_H */
