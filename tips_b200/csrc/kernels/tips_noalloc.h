/* Entry point of the kernel library for callers that must not allocate device memory.
 *
 * It has no counterpart in the reference, which has no device code at all.
 *
 * Who needs it: code that runs where an allocation is not allowed or not possible, for example
 * inside a region that has been handed a fixed memory budget, from a host thread that may not touch
 * the allocator of the framework that owns the process (a data-loader or communication thread calling
 * this library next to PyTorch's caching allocator), or late in a job when device memory is fully
 * committed and a failed cudaMalloc would abort the step.  Such a caller still owns its inputs and
 * outputs; what it cannot provide is the scratch buffer that the batch-norm forward needs for its
 * per-block partial sums.
 *
 * tipsk_bn_fwd_train_noalloc is tipsk_bn_fwd_train with that scratch taken from a fixed array that
 * lives inside the library's device image (a file-scope `static __device__` array of
 * TIPSK_BN_NOALLOC_SCRATCH_FLOATS floats, 3 MiB, held by every GPU that loads the library until the
 * process exits).  It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 *  - Limit: 2 * c * tipsk_bn_partials(m, c) must not exceed TIPSK_BN_NOALLOC_SCRATCH_FLOATS; larger
 *    problems are rejected with a negative return code and a message in tipsk_last_error().
 *  - The first call on each device looks up the device address of the array (cudaGetSymbolAddress,
 *    with that device current) and caches it.  Make that first call outside any stream capture.
 *  - All calls share the one array.  The kernel writes every partial sum before it reads it, so stale
 *    contents from an earlier call are harmless and nothing has to be cleared; but two calls that
 *    overlap on the GPU (different streams, no ordering between them) race on the array.  Order them.
 */
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TIPSK_BN_NOALLOC_SCRATCH_FLOATS (768 * 1024)

/* Same arguments and semantics as tipsk_bn_fwd_train, minus the workspace pointer. */
int tipsk_bn_fwd_train_noalloc(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                               float* running_mean, float* running_var, float* save_mean, float* save_invstd,
                               int64_t m, int c, float eps, float momentum, int relu, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
