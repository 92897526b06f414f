// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in divedb/InferX; it exists for programs
// that embed this library where cudaMalloc is off limits: a serving process that
// handed the whole device to its own arena at start-up and has nothing left for
// a driver allocation, or a step loop that may not call anything that
// synchronises the device or can fail for lack of memory half-way through a
// request.  The ordinary entry point, ix_paged_attention_decode, expects the
// caller to bring two scratch buffers for the split-KV partial results; this
// variant brings its own, a fixed array inside the library.
//
// Limit: the partial results need S * heads * splits * (head_dim + 2) floats,
// where splits = ix_attn_decode_splits(S, heads, kv_heads, max_kv_len).  The
// built-in array holds IX_NOALLOC_SCRATCH_FLOATS floats (4 MiB); a call that
// needs more returns IX_ERR_SCRATCH_TOO_SMALL, prints one line to stderr saying
// how much was needed, and launches nothing.  The array is part of the library's
// device image, so every GPU that loads the library keeps these 4 MiB until the
// process exits.
//
// Set-up: the first call on each device looks up the array's device address
// (with that device current) and remembers it.  Make that first call before any
// stream capture on that device.
//
// Sharing: all calls on a device use the same array, and it keeps what the last
// call left in it.  Nothing in it has to start at zero (every partial a call
// reads was written by that same call), but two calls that overlap on the GPU
// (different streams without an ordering between them) overwrite each other's
// partial results.  Run them on one stream, or order them with events.
//
// The function itself calls no cudaMalloc, cudaFree or any other allocating
// routine; inputs and the output are the caller's, as with the ordinary entry.
#pragma once
#include <cuda_runtime.h>

#define IX_NOALLOC_SCRATCH_FLOATS (1u << 20)
#define IX_ERR_SCRATCH_TOO_SMALL (-6)

#ifdef __cplusplus
extern "C" {
#endif

// q [S, heads, head_dim], caches [pages, kv_heads, page_size, head_dim], block
// table [S, max_blocks], kv_len [S] (the query of sequence s sits at position
// kv_len[s] - 1), out [S, heads, head_dim]; act_dtype 0 = float32, 1 = bfloat16.
// max_kv_len is an upper bound on kv_len[], used to choose the number of splits.
// Returns 0, a positive cudaError_t, or a negative IX_ERR_* code.
int ix_paged_attention_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                      const int* block_table, const int* kv_len, void* out,
                                      int act_dtype, int S, int heads, int kv_heads, int head_dim,
                                      int page_size, int max_blocks, int window, float scale,
                                      int max_kv_len, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
