// Attention over a paged cache for callers that must not allocate device memory.
//
// This entry point has no counterpart in MiniServe-LLM-NV; it exists for users of this library
// whose code runs where cudaMalloc is off limits: inside another application's memory pool, in a
// latency-critical loop that may not enter the allocator, or in a process that gave all device
// memory away when it started.  They still pass their own inputs and outputs; what the library
// needs beyond those (the partial results of the key splits) lives in an 8 MiB array that is part
// of the library image on every GPU that loads it, from load until the process exits.
//
// It computes exactly what ms_paged_attention_mma computes for a step of single tokens (one new
// token per request, bfloat16, head size 32, 64 or 128), with the keys of each request split into
// `num_splits` parts that run in parallel and are merged at the end.
//
//  * Limit: n_tokens * n_q * num_splits * (d + 1) must not exceed 2,097,152 floats; a larger
//    request is refused with a message (ms_last_error) and nothing is launched.
//  * The first call on a device looks up that device's address of the array (the device must be
//    current) and remembers it.  Make that first call before any stream capture begins.
//  * All calls share the one array, and it keeps what the last call left in it.  Nothing in it has
//    to be cleared between calls, but two calls whose kernels may run at the same time on the GPU
//    (different streams without an ordering between them) overwrite each other's partial results:
//    order such calls yourself.
//  * It calls no cudaMalloc, cudaFree or other allocating routine.
//
// Returns 0 on success.  Arguments as for ms_paged_attention_mma: q, out [n_tokens, n_q, d]
// bfloat16; k_pool, v_pool [pages, n_kv, page_size, d] bfloat16; block_tables [n_requests,
// table_stride], query_start [n_requests + 1], context_lens [n_requests] int32, all on the device.
#pragma once
#include <cuda_runtime.h>

extern "C" int ms_paged_attention_decode_static(const void* q, const void* k_pool, const void* v_pool,
                                                const int* block_tables, int table_stride, const int* query_start,
                                                const int* context_lens, int page_size, int n_q, int n_kv, int d,
                                                float scale, int window, void* out, int num_splits, int n_requests,
                                                int n_tokens, cudaStream_t stream);
