// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for embedders of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits - inside a host program that hands this
// library a fixed memory budget and audits every allocation, under a real-time loop where an allocation's
// latency (or its implicit device synchronisation) is unacceptable, or from a plugin that only receives
// device pointers from its host and has no allocator of its own.  The ordinary entry point
// `hk_attention_flash` needs two scratch buffers for the partial results of split key ranges, which its
// caller allocates.  `hk_attention_decode_noalloc` runs the same decode kernel and the same combine kernel,
// but keeps those partials in a fixed array that is part of the library image.
//
// Limits and rules:
//   * The scratch is HK_NOALLOC_SCRATCH_BYTES (4 MiB) of device memory per GPU, held by every GPU that loads
//     this library until the process exits.  A call needs n_parts * G * 16 * (hd + 2) * 4 bytes of it; a call
//     that needs more is refused with HK_ERR_SCRATCH_TOO_SMALL and launches nothing.
//   * The first call on a device resolves the array's device address (cudaGetSymbolAddress, with that device
//     current).  Make that first call outside any stream capture.
//   * All calls share the one array, and it keeps what the last call left.  Nothing in it has to start at
//     zero: every partial a call reads was written by that same call.  Two calls that overlap on the GPU
//     (different streams without an ordering between them) race on the array; order them.
//   * The function calls no cudaMalloc/cudaFree and no allocating library routine; inputs, outputs, the work
//     items and the per-token combine tables are the caller's device buffers.
#pragma once

#define HK_NOALLOC_SCRATCH_BYTES (4u << 20)
#define HK_ERR_SCRATCH_TOO_SMALL 100002

#ifdef __cplusplus
extern "C" {
#endif

// Decode attention over the paged cache with split key ranges (the `nw = 1` variant of hk_attention_flash
// followed by hk_attention_combine).  Arguments as there: `items` [n_items][8] int32 work items, of which
// those with part >= 0 write partial number `part` (0 <= part < n_parts); `first`, `count`, `row0` [n_tokens]
// int32 say which partials each token merges.  Returns 0, a cudaError_t, HK_ERR_UNSUPPORTED (100001) for
// shapes the kernel refuses, or HK_ERR_SCRATCH_TOO_SMALL.
int hk_attention_decode_noalloc(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                int table_stride, const void* items, int n_items, int n_parts, const int* first,
                                const int* count, const int* row0, void* out, int n_tokens, int H, int G, int hd,
                                int page_tokens, int window, float scale_log2, int pages_cap, void* stream);

#ifdef __cplusplus
}
#endif
