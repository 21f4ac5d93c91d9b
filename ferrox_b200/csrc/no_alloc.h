// An entry point for callers that cannot allocate device memory.
//
// This declaration has no counterpart in the reference (antonellof/ferrox): it exists
// for users of this library who run where cudaMalloc is not an option, for example
// code that executes inside a region where the allocator must not be entered (a
// callback on a stream, a real-time loop with a fixed memory budget, a host that
// handed all device memory to another pool up front) and that therefore cannot
// provide the scratch buffers fx_decode_attention asks for.
//
// fx_decode_attention_noalloc computes exactly what fx_decode_attention computes
// (attention of a few query tokens over paged keys and values, split over key
// ranges and merged), with the caller passing only inputs and outputs.  The
// per-split partial results are kept in a fixed array inside the library.
//
//  * Limit: n_tokens * n_heads * n_splits * (head_dim + 2) must not exceed
//    FX_NOALLOC_SCRATCH_FLOATS (2,097,152 floats = 8 MiB); larger requests return
//    FX_ERR_SCRATCH (-5) and launch nothing.  Each GPU on which the library is used
//    holds these 8 MiB until the process exits.
//  * The first call on a device looks up the array's device address (that device
//    must be current).  Make this first call outside any stream capture.
//  * The call itself calls no cudaMalloc, cudaFree or allocating library routine.
//  * The call assumes nothing about the kernels launched before it on the stream:
//    its kernels read nothing (queries, positions, block table, keys, values) until
//    those have finished, however many positions they wrote.
//  * All calls share the one array, and it keeps the previous call's contents.
//    Nothing needs clearing between calls (every value read is written first by the
//    same call), but two calls whose kernels overlap on the GPU (different streams,
//    or one stream per thread) race on it: issue them on one stream, or order them.
#pragma once

#define FX_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define FX_ERR_SCRATCH -5   // the request needs more scratch than the fixed array holds

#ifdef __cplusplus
extern "C" {
#endif

int fx_decode_attention_noalloc(const void* q, long ldq, const void* k_pages, const void* v_pages, int dtype,
                                const int* block_table, int table_width, int page_size, const int* positions,
                                const int* token_seq, const int* seq_slot, void* out, long ldo, int n_tokens,
                                int n_heads, int n_kv_heads, int head_dim, int window, float scale, int split_len,
                                int n_splits, void* stream);

#ifdef __cplusplus
}
#endif
