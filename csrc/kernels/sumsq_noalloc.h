// Sum of squares of an fp32 vector for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists only in this library.
//
// Who needs it: code that runs where cudaMalloc / cudaFree (or any allocating library routine,
// torch's caching allocator included) must not be called — for instance a host thread that is
// inside a region the application has declared allocation-free, a plug-in loaded by a process that
// owns all device memory itself and hands out only input/output buffers, or a latency-critical
// loop in which an implicit device synchronisation caused by cudaFree would be unacceptable.
// The regular entry point bb_sumsq() needs a caller-provided scratch buffer for its per-block
// partial sums; such callers have nowhere to get one from.
//
// How it works: the partial sums live in a fixed array that is part of the library image itself
// (file-scope `static __device__`, BB_SUMSQ_NOALLOC_SCRATCH_FLOATS floats = 4 KiB).  Every GPU on
// which the library is loaded holds that array until the process exits.
//
// Limits and rules:
//   * n must be in [0, BB_SUMSQ_NOALLOC_MAX_ELEMS]; larger inputs are rejected with
//     BB_SUMSQ_NOALLOC_ESIZE and a message on stderr, nothing is launched.
//   * `g` must be 16-byte aligned; `out` is one float in device memory supplied by the caller.
//   * The first call on each device looks up the device address of the scratch array
//     (cudaGetSymbolAddress).  Make that first call before starting any stream capture on that
//     device.  First calls made by several host threads at once are safe (the cached address is
//     an atomic and every thread would store the same value).
//   * All calls on a device share the one scratch array, which still holds the previous call's
//     partial sums when the next call starts (every slot that is read is rewritten first, so no
//     clearing is needed).  Two calls whose kernels overlap on the GPU — different streams, or
//     different host threads without ordering — race on it and give wrong sums.  Order them.
//   * Nothing here calls cudaMalloc, cudaFree, or any routine that allocates.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define BB_SUMSQ_NOALLOC_SCRATCH_FLOATS 1024
#define BB_SUMSQ_NOALLOC_MAX_ELEMS (1L << 28) /* 268,435,456 floats = 1 GiB of input */
#define BB_SUMSQ_NOALLOC_ESIZE (-3)           /* n outside [0, MAX_ELEMS] */
#define BB_SUMSQ_NOALLOC_EARG (-1)            /* null / misaligned pointer */
#define BB_SUMSQ_NOALLOC_ESETUP (-5)          /* scratch address lookup failed on this device */

// out[0] = sum(g[i]^2) (accumulate == 0) or out[0] += sum (accumulate != 0), on `stream`.
// Returns 0, one of the negative codes above, or a positive cudaError_t from the launch.
int bb_sumsq_noalloc(const float* g, long n, float* out, int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
