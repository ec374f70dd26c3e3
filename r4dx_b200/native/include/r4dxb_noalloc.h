/* Entry point for callers that cannot allocate device memory.
 *
 * This has no counterpart in the reference engine; it exists for embedders of this library that
 * are handed device pointers by someone else and have no allocator of their own to ask: code that
 * runs inside another runtime's callback or plugin hook where cudaMalloc is forbidden, and code
 * that sits inside a CUDA-graph capture, where an allocation would break the capture.  Such a
 * caller can provide the logits and the result arrays (it owns those) but not the temporary
 * buffer that r4dxb_argmax_rows needs for its per-part partial results.
 *
 * r4dxb_argmax_rows_static is r4dxb_argmax_rows with that temporary buffer taken from a fixed
 * 128 KiB array that is part of the library image on every GPU that loads it:
 *
 *   - at most R4DXB_ARGMAX_STATIC_MAX_ROWS rows per call; more returns R4DXB_TOO_LARGE and
 *     launches nothing;
 *   - the call allocates nothing and frees nothing (no cudaMalloc, no cudaFree, no library
 *     routine that allocates);
 *   - the first call on each device looks up the array's device address (a host-side query,
 *     done with that device current).  Make that first call during start-up, before any stream
 *     capture begins on that device; later calls only launch kernels;
 *   - all calls on a device share the one array.  Each call overwrites every slot it later
 *     reads, so leftovers of earlier calls are harmless, but two calls whose kernels may run at
 *     the same time on one device (different streams, or different host threads without
 *     ordering) race on it and can return wrong indices.  Order such calls on one stream or
 *     with events.
 *
 * Results (ids with ties to the lowest index, plus id_offset; optional max values) are identical
 * to r4dxb_argmax_rows. */
#ifndef R4DXB_NOALLOC_H_
#define R4DXB_NOALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

#define R4DXB_ARGMAX_STATIC_MAX_ROWS 64

int r4dxb_argmax_rows_static(const void* logits, int is_f32, int T, int V, int id_offset, int* out_ids,
                             float* out_vals, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* R4DXB_NOALLOC_H_ */
