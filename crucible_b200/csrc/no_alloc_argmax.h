/* Greedy token choice for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference; it exists for hosts of
 * this library that cannot call cudaMalloc: code that runs while a CUDA graph
 * is being captured on another stream of the same context, code inside a
 * memory-pool owner that forbids foreign allocations, or a latency-critical
 * loop whose device memory is budgeted to the byte up front.  The library's
 * usual argmax (cb_argmax_rows) takes a scratch buffer from its caller, which
 * for those hosts means one more allocation to plan; this variant carries its
 * scratch with the library instead.
 *
 * It computes, for each of n_rows rows of fp32 logits [n_rows, vocab], the index
 * of the highest value (lowest index among equals; a NaN displaces nothing and a
 * NaN in column 0 is never displaced, so such a row gives 0), exactly as
 * cb_argmax_rows does, in two kernels: per-slice
 * maxima into scratch, then the maximum over the slices.
 *
 * Scratch: a file-scope device array inside the library, 64 KiB, enough for
 * CB_ARGMAX_STATIC_MAX_ROWS rows.  Every GPU that loads the library holds those
 * 64 KiB until the process exits.  All calls share the array: two calls whose
 * kernels overlap on the GPU (different streams, no ordering between them) race
 * on it and may both return wrong ids; order them on one stream or with events.
 * Nothing in the array has to start at zero: each call overwrites every entry it
 * later reads, so stale contents of an earlier call are harmless.
 *
 * Every call, not only the first, must be made with the logits' device current:
 * the scratch address is chosen by cudaGetDevice at each call.  The first call
 * on a device also looks up the array's device address (one
 * cudaGetSymbolAddress with that device current); make that first call before
 * any stream capture begins.  No call allocates or frees anything: no
 * cudaMalloc, cudaFree, or library routine that allocates.
 *
 * Returns 0 on success, CB_ERR_STATIC_TOO_LARGE if n_rows exceeds
 * CB_ARGMAX_STATIC_MAX_ROWS (nothing is launched), otherwise the cudaError_t of
 * the failing runtime call.  `stream` is a cudaStream_t. */
#pragma once

#define CB_ARGMAX_STATIC_MAX_ROWS 256
#define CB_ERR_STATIC_TOO_LARGE 100002

#ifdef __cplusplus
extern "C"
#endif
int cb_argmax_rows_static(const float* logits, int n_rows, int vocab, int* out_ids, void* stream);
