/* Entry points of libcoffin_b200.so that never allocate.
 *
 * This header has no counterpart in the reference engine; it exists for callers of this library
 * that are not in a position to allocate device memory at the time they need a result:
 *   - a serving loop that sized every buffer at start-up and runs with the allocator frozen,
 *     so that a late cudaMalloc cannot fail (or stall on an implicit device synchronisation)
 *     in the middle of a decode step;
 *   - code that is driven from inside someone else's runtime (a plugin, a callback, a sandboxed
 *     worker) where the host owns all device memory and a private allocation is not allowed.
 * The ordinary entry point, cb_argmax, needs a caller-provided scratch buffer for its two-stage
 * reduction; the Python wrapper allocates that buffer on first use.  The variant below carries its
 * scratch inside the library instead.
 *
 * int cb_argmax_static(const void* logits, void* out, int64_t M, int64_t V, int64_t ld, void* stream)
 *
 *   logits  device pointer, fp32, M rows of V values, row pitch ld (elements)
 *   out     device pointer, int64, M entries: index of the row maximum (lowest index on ties)
 *   M       rows, 0 <= M <= cb_argmax_static_max_rows() (64); larger M is rejected with
 *           CB_ERR_SHAPE (10001) and nothing is launched - use cb_argmax with your own scratch
 *   stream  cudaStream_t the kernel is launched on
 *   returns 0 on success, a cudaError_t value or a CB_ERR_* code otherwise
 *
 * Properties and limits:
 *   - No call allocates or frees: no cudaMalloc, cudaFree, or allocating library routine.
 *   - The scratch is one file-scope device array of about 50 KB.  Every GPU on which the library is
 *     loaded holds it until the process exits.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current) and clears it with a cudaMemsetAsync on the given stream.  Make that
 *     first call before any stream capture begins.
 *   - All calls on a device share the one array.  Two calls that can overlap on the GPU (different
 *     streams, no dependency between them) race on it and may return wrong indices; order them
 *     on one stream or with events.  The array keeps the previous call's partial results; the only
 *     state that must be zero between calls, the arrival tickets, is re-armed by the kernel itself.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int cb_argmax_static(const void* logits, void* out, int64_t M, int64_t V, int64_t ld, void* stream);
int64_t cb_argmax_static_max_rows(void);

#ifdef __cplusplus
}
#endif
