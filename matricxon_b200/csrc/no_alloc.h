// Paged attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (nesmind/matricxon has no GPU code at
// all); it exists for hosts that embed this library where cudaMalloc is off limits: a plugin
// running inside another framework's memory pool, a real-time loop that may not take the
// allocator's locks or trigger an implicit device synchronisation, a process whose memory
// budget was fixed and handed out at start-up. Such a caller still owns its inputs and its
// output; what it cannot provide is the scratch buffer that split-key attention needs for
// its per-split partial results.
//
// mx_paged_attention_static is mx_paged_attention with that scratch taken from a fixed
// array inside the library image instead of from the caller:
//
//   * the array holds MX_STATIC_ATTENTION_SCRATCH_BYTES (8 MiB) and is reserved on every GPU
//     that loads the library, from load until the process exits, whether or not it is used;
//   * a call whose partials would not fit (tokens * heads * splits * (head_dim + 2) * 4 bytes
//     above the limit) is refused with MX_ERR_UNSUPPORTED and a message; nothing is launched;
//   * the first call on each device looks the array's device address up
//     (cudaGetSymbolAddress) and remembers it; make that first call outside any stream
//     capture. Later calls only launch kernels;
//   * the array that is used is the one of the device that is current when the call is made:
//     `q`, `out`, `cache`, the index arrays and `stream` must all belong to that device. A
//     caller that holds pointers of device 1 while device 0 is current gets device 0's array,
//     which device 1's kernels cannot be assumed to reach: set the device first;
//   * the function calls no cudaMalloc, cudaFree or allocating library routine;
//   * every call uses the same array and leaves its partials there. The kernels write each
//     partial before the merge reads it, so nothing needs clearing between calls, but two
//     calls that overlap on the GPU (different streams, or one stream captured and replayed
//     concurrently) race on the array. Serialise them.
//
// Arguments are those of mx_paged_attention without `scratch`.
#pragma once

#include <cuda_runtime.h>

#define MX_STATIC_ATTENTION_SCRATCH_BYTES (8ll * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int mx_paged_attention_static(const void* q, int dtype, int q_stride, const void* cache,
                              long long n_pages, int page_size, const int* block_tables,
                              int bt_stride, const int* tok_seq, const int* positions,
                              int n_tokens, int n_heads, int n_kv_heads, int head_dim, int window,
                              float scale, void* out, int out_stride, int n_splits, int* status,
                              cudaStream_t stream);

// The limit above, for callers that size their splits against it.
long long mx_static_attention_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
