/* One extra entry point of libtinyserve_b200: paged split-K decode attention that allocates
 * nothing.
 *
 * It has no counterpart in the reference engine (princemittalr/tinyserve); it exists for
 * callers of this library that are not allowed to allocate device memory when they call it:
 * code that runs inside a region where cudaMalloc is forbidden or would deadlock (a stream
 * capture, a callback, a real-time loop with a fixed memory plan) and code that is handed a
 * fixed set of buffers by a host framework and has no allocator of its own. The regular entry
 * point (ts_paged_attention_simt) asks its caller for two scratch buffers that hold the
 * partial results of the key ranges; this one keeps that scratch in a fixed array inside the
 * library instead, so the caller passes inputs and outputs only.
 *
 * Limits and rules:
 *  - The scratch is TS_STATIC_SCRATCH_FLOATS floats (8 MiB). Every GPU on which the library
 *    is loaded holds that much from load until the process exits. A call needs
 *    num_decode * num_heads * num_splits * (head_dim + 2) floats; a call that needs more is
 *    refused with TS_ERR_SCRATCH_TOO_SMALL and launches nothing.
 *  - The first call on each device looks up the array's device address once (with that
 *    device current). Make that first call outside any stream capture.
 *  - All calls share the one array, and it keeps what the last call left in it. The kernels
 *    overwrite every element they later read, so nothing needs clearing; but two calls that
 *    run on the GPU at the same time (different streams, no dependency) would race on it.
 *    Order them on one stream or with an event.
 *  - num_splits is at most TS_STATIC_SCRATCH_MAX_SPLITS (32, the limit of every decode launcher of
 *    the library: the merge of the ranges stages two floats per range and head in shared memory
 *    sized for that many); more is refused with TS_ERR_BAD_ARGUMENT (-1) and launches nothing.
 *  - Neither this function nor anything it calls allocates or frees device memory.
 *
 * Arguments are those of ts_paged_attention_simt for the decoding requests: q and out are
 * [tokens, num_heads, head_dim], the caches [pages, num_kv_heads, page_size, head_dim],
 * block_tables [requests, table_width] int32, cu_q [requests + 1], ctx_lens [requests],
 * decode_seqs lists the num_decode requests (each brings exactly one token). dtype: 0 = float,
 * 1 = bfloat16. Returns 0, a negative TS_ERR_* code, or a positive cudaError_t.
 */
#pragma once
#include <cuda_runtime.h>

#define TS_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define TS_ERR_SCRATCH_TOO_SMALL (-3)
#define TS_STATIC_SCRATCH_MAX_SPLITS 32

#ifdef __cplusplus
extern "C" {
#endif

int ts_decode_attention_static_scratch(const void* q, void* out, const void* k_cache, const void* v_cache,
                                       const int* block_tables, int table_width, const int* cu_q,
                                       const int* ctx_lens, const int* decode_seqs, int num_decode,
                                       int num_heads, int num_kv_heads, int head_dim, int page_size,
                                       float scale, int window, int num_splits, int dtype,
                                       cudaStream_t stream);

/* How many floats a call with these sizes needs (to check against TS_STATIC_SCRATCH_FLOATS). */
long long ts_decode_attention_static_scratch_need(int num_decode, int num_heads, int head_dim, int num_splits);

#ifdef __cplusplus
}
#endif
