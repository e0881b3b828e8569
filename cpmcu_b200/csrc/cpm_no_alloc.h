// Declaration of the one entry point of this library that allocates nothing.
//
// It has no counterpart in OpenBMB/CPM.cu; it exists for callers of this library that
// cannot allocate device memory at the point where they need attention: code that runs
// inside a region where cudaMalloc is forbidden or would stall (a latency-critical
// serving loop that must not touch the allocator, a host that pre-reserved all device
// memory for its own pools, a plug-in loaded into a process whose allocator it may not
// call).  Every other entry point of the library takes its scratch memory from the
// caller; this one brings its own.
//
// cpm_decode_attention_bf16_static computes the same result as
// cpm_decode_attention_bf16: attention of one query token per sequence over that
// sequence's pages of the key-value cache (bf16, grouped-query heads, the keys split into
// n_splits shares whose partial results are combined).  The partial results live in a
// file-scope device array of CPM_STATIC_SCRATCH_FLOATS floats (16 MiB) that every GPU
// which loads the library holds until the process exits.
//
// Rules for callers:
//  * Sizes: n_seqs * n_kv * ceil(heads_per_kv / 16) * n_splits * (16 * d + 32) floats must
//    fit into CPM_STATIC_SCRATCH_FLOATS; otherwise nothing is launched, CPM_STATIC_TOO_LARGE
//    is returned and error_text (if given) says how much was asked for.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress) with that device current; make that first call outside any
//    stream capture.  Later calls on the device reuse the address.
//  * All calls share the one array per device.  It keeps the previous call's contents;
//    every element a call reads it has written before in the same call, so nothing needs
//    clearing, but two calls that overlap on the GPU (different streams without ordering,
//    or different host threads) race on it.  Order them.
//  * The call does not allocate: no cudaMalloc, no cudaFree, no allocating library routine.
//    Inputs and outputs are the caller's device buffers as for cpm_decode_attention_bf16.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define CPM_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define CPM_STATIC_TOO_LARGE (-2)
#define CPM_STATIC_SETUP_FAILED (-3)

#ifdef __cplusplus
extern "C" {
#endif

// q, out: [n_seqs, n_heads, d] bf16.  k_cache: pages [page][kv_head][64][d] bf16; v_cache: pages
// [page][kv_head][d][64] bf16.  kv_len, slots: int32 [n_seqs]; page_table: int32 [slots][max_pages].
// d is 32, 64, 96 or 128.  Returns 0 when both kernels were launched on ``stream``; -1 for sizes the
// kernels do not take; CPM_STATIC_TOO_LARGE; CPM_STATIC_SETUP_FAILED; or a positive CUDA error.
// error_text (may be null) receives a zero-terminated message of at most error_text_len bytes.
__attribute__((visibility("default")))
int cpm_decode_attention_bf16_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                     const int* kv_len, const int* slots, const int* page_table, int max_pages,
                                     int n_seqs, int n_heads, int n_kv, int d, int n_splits, float scale,
                                     cudaStream_t stream, char* error_text, int error_text_len);

#ifdef __cplusplus
}
#endif
