/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in pytorch-labs/gpt-fast: it is an
 * addition of this library.
 *
 * Who needs it: code that runs where cudaMalloc must not be called, for
 * example a plug-in loaded into a host process that owns all device memory
 * and hands out fixed buffers, a real-time loop that may not block on the
 * allocator, or a runtime whose memory pool is closed after start-up.  Such a
 * caller can still pass its own input and output buffers, but it has nowhere
 * to get the scratch memory that the split-KV decode kernel needs for the
 * per-slice partial results.
 *
 * gfb_attn_decode_noalloc is gfb_attn_decode (attention_bf16.cu) with that
 * scratch taken from a fixed array that lives in the library's own device
 * image (file scope, `static __device__`), so the call allocates nothing: no
 * cudaMalloc, no cudaFree, no allocating library routine.
 *
 * Limits and rules:
 *  - The array holds GFB_NOALLOC_SCRATCH_FLOATS floats (4 MiB).  Every GPU
 *    whose context loads this library keeps that much memory until the
 *    process exits.  A call needs n_tokens * H * splits * (d + 2) floats;
 *    a larger request is refused with an error (gfb_last_error() says so),
 *    nothing is launched.  With splits == 1 no scratch is used at all.
 *  - The first call on a device looks up the array's device address
 *    (cudaGetSymbolAddress, once per device, with that device current) and
 *    remembers it.  Make that first call outside any stream capture.
 *  - All calls share the one array, and it keeps whatever the previous call
 *    left in it.  Nothing in it has to start at zero: every slot that the
 *    merge step reads is written first by the same call (slices without keys
 *    write an empty partial).  But two calls that overlap on the GPU (two
 *    streams, or two host threads) would write the same words: run calls of
 *    this entry point one after another on one stream, or order them with
 *    events.
 *
 * Arguments are those of gfb_attn_decode without `scratch`.  Returns 0 on
 * success.
 */
#pragma once
#include <cuda_runtime.h>

#define GFB_NOALLOC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

int gfb_attn_decode_noalloc(const void* q, void* out, void* k_pool, void* v_pool, const int* page_table, int max_pages,
                            int page_size, int n_pages, const int* cu_seqlens, const int* tok_seq, const int* slots,
                            const int* lengths, int n_seqs, int n_tokens, int H, int G, int d, float scale, int window,
                            int splits, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
