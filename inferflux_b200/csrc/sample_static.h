/* Token sampling for callers that may not allocate device memory.
 *
 * This entry point has no counterpart in vjsingh1984/inferflux; it is an
 * addition of this library.
 *
 * Who needs it: code that runs where cudaMalloc is off limits.  Examples are a
 * host program that hands this library a fixed memory budget and forbids any
 * further allocation (an embedded or real-time loop, a plugin inside another
 * engine's memory pool), and a sampler called between the steps of someone
 * else's captured work, where an allocation would synchronise the device or
 * fail outright.  The regular entry point, ifx_sample, wants a scratch buffer
 * of n_rows * vocab floats from its caller; a caller that cannot allocate has
 * nowhere to get one.
 *
 * ifx_sample_static does the same work with the scratch inside the library: a
 * file-scope device array of IFX_SAMPLE_STATIC_MAX_ROWS *
 * IFX_SAMPLE_STATIC_MAX_VOCAB floats (8 MiB).  Every GPU that loads the library
 * holds that array from load until the process exits, whether or not the entry
 * point is ever called.  The caller still passes the logits, the per-row
 * parameters and the output.
 *
 * Rules of use
 *  - n_rows <= IFX_SAMPLE_STATIC_MAX_ROWS and vocab <= IFX_SAMPLE_STATIC_MAX_VOCAB,
 *    otherwise IFX_ERR_STATIC_TOO_LARGE is returned and nothing is launched
 *    (ifx_sample_static_message() gives the text).
 *  - The first call on a device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) and remembers it.  Make
 *    that first call outside any stream capture.
 *  - All calls on a device share the one array, and it keeps whatever the last
 *    call left in it.  Nothing in it has to start at zero: a call overwrites
 *    every element it later reads.  Two calls that overlap on the GPU (two
 *    streams, or two host threads) race on it; run them one after the other.
 *  - No cudaMalloc, cudaFree or other allocating routine is called, here or in
 *    the kernel.
 *
 * Arguments are those of ifx_sample without `weights`.  The kernel is the one
 * ifx_sample uses for rows too long for a cluster's shared memory; for shorter
 * rows ifx_sample runs a kernel that needs no scratch and adds masses as
 * integers, and the two return the same token unless the row's uniform falls
 * within float32 rounding of a boundary between two tokens.  Returns 0 on
 * success, a cudaError_t value for a CUDA failure, or one of the codes below.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IFX_SAMPLE_STATIC_MAX_ROWS 8
#define IFX_SAMPLE_STATIC_MAX_VOCAB 262144
#define IFX_ERR_STATIC_TOO_LARGE 100003

__attribute__((visibility("default")))
int ifx_sample_static(const float* logits, long long row_stride, const float* temperature, const int* top_k,
                      const float* top_p, const float* min_p, const unsigned long long* seeds,
                      const unsigned long long* counters, int* out, int n_rows, int vocab, cudaStream_t stream);

/* Text for a code returned by ifx_sample_static (a static string; never NULL). */
__attribute__((visibility("default")))
const char* ifx_sample_static_message(int code);

#ifdef __cplusplus
}
#endif
