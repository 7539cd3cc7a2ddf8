// Flash-decoding for callers that cannot allocate device memory.
//
// This entry point has no counterpart in beyondHJM/tinyinfer.cpp; it exists for this library's
// own users.  `ti_attn_decode` wants two scratch buffers from its caller (the partial results of
// the key splits).  Some callers have no way to provide them: a host program that has handed
// every byte of the device to its own pool and forbids cudaMalloc afterwards, a plain C caller
// that links this library without a tensor library's allocator, or a latency-critical loop in
// which an allocation (which may synchronise the device) is not acceptable.  For them
// `ti_attn_decode_noalloc` keeps the scratch in a fixed array inside the library.
//
// What to know before using it:
//  * The array is TI_DECODE_NOALLOC_SCRATCH_BYTES (8 MiB) of device memory per GPU that loads
//    the library, held until the process exits.  A call that needs more is refused with an
//    error message (see ti_last_error) and launches nothing.  The need is
//    num_rows * num_heads * num_splits * (head_dim + 2) * 4 bytes.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, once
//    per device, with that device current).  Make that first call before any stream capture.
//  * The entry point itself calls no cudaMalloc, cudaFree or other allocating routine.
//  * All calls share the one array, and it keeps what the last call left.  Nothing in it has to
//    start at zero: every slot a call reads it has written itself.  Two calls whose kernels can
//    overlap on the GPU (different streams, no dependency between them) race on the array; keep
//    calls on one stream or order them with events.
//  * Inputs and outputs are the caller's, as for ti_attn_decode; arguments have the same meaning.
#pragma once

#define TI_DECODE_NOALLOC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int ti_attn_decode_noalloc(const void* q, const int* rows, int num_rows, const int* positions,
                           const int* req_of_tok, const int* block_table, int bt_stride,
                           const void* pages, int num_pages, int page_size, int num_heads,
                           int num_kv_heads, int head_dim, int window, float scale, int num_splits,
                           void* out, int* status, void* stream);

#ifdef __cplusplus
}
#endif
