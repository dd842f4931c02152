// Ask the memory system to bring ranges of global memory into L2 ahead of their use
// (cp.async.bulk.prefetch.L2): a decode step reads every weight exactly once, one kernel after
// the other, and the attention kernel in the middle of a layer leaves part of the memory
// bandwidth idle; the weights that the products after it will stream are fetched meanwhile.
// The kernel only issues the requests (one thread per piece) and ends; nothing waits for the
// data, and nothing goes wrong if a line is evicted again before its use. No counterpart in
// upstream, whose products are library calls.
#include "common.cuh"
#include "prefetch.cuh"

namespace ts {

// Bytes per request: prefetch.cuh. The kernel lasts until its requests are served, and an
// SM passes them on at about 0.15 TB/s, so the number of CTAs sets the rate: 16 KB x 128 threads
// fetches 23 MB with 12 CTAs at 1.9 TB/s in 11 us. How long the kernel beside it lasts depends on
// the step, so the caller chooses the number of requests per CTA (`threads`, 16 to 128): fewer per
// CTA means more CTAs and a proportionally higher rate.
// The kernel runs on a stream of its own, forked before the kernel it runs beside and joined after
// it. Two other placements were measured in the recorded decode step (B200, Qwen3-0.6B sizes, batch
// 8: 0.92 ms a step as it is) and are worse: the attention kernel's own CTAs issuing the requests
// (1.06 ms: a CTA lasts until its requests are served, and those CTAs are the step's critical
// path), and this kernel as a link of the same stream's chain of programmatically launched kernels,
// behind the attention kernel, waiting for it at its end (1.02 ms: it starts later, and the product
// after it waits for its end).
__global__ void prefetch_l2_kernel(PrefetchRanges r) { prefetch_piece(r, blockIdx.x * blockDim.x + threadIdx.x); }

// The pages of a paged cache that the listed requests hold, for the keys and for the values: thread
// (request, page of its table, keys | values, piece) asks for one piece of its page, if the
// request's context reaches that page. Block tables and lengths are read on the device, so the
// kernel can be part of a recorded step.
__global__ void prefetch_pages_kernel(const char* k_base, const char* v_base, unsigned long long page_bytes,
                                      const int* __restrict__ block_tables, int table_width,
                                      const int* __restrict__ ctx_lens, int num_seqs, int page_size, int pieces_per_page) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int piece = (int)(idx % pieces_per_page);
  const int which = (int)((idx / pieces_per_page) & 1);
  const long long bp = idx / (2 * pieces_per_page);
  const int p = (int)(bp % table_width), b = (int)(bp / table_width);
  if (b >= num_seqs || p * page_size >= ctx_lens[b]) return;
  const int page = block_tables[(size_t)b * table_width + p];
  const unsigned long long off = (unsigned long long)piece * PF_PIECE;
  const unsigned long long left = page_bytes - off;
  const unsigned int n = left < PF_PIECE ? (unsigned int)left : PF_PIECE;
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"((which ? v_base : k_base) + (unsigned long long)page * page_bytes + off), "r"(n) : "memory");
}

}  // namespace ts

using namespace ts;

// Prefetch into L2 the cache pages (keys and values, `page_bytes` each, 16-byte aligned) that the
// first `num_seqs` requests of `block_tables` [*, table_width] hold up to their `ctx_lens`.
extern "C" int ts_prefetch_pages(const void* k_cache, const void* v_cache, unsigned long long page_bytes,
                                 const int* block_tables, int table_width, const int* ctx_lens, int num_seqs,
                                 int page_size, int threads, cudaStream_t stream) {
  if (num_seqs <= 0 || table_width <= 0) return 0;
  if (threads < 16 || threads > 128 || threads % 16 != 0 || page_size <= 0) return TS_ERR_BAD_ARGUMENT;
  if ((((uintptr_t)k_cache) | ((uintptr_t)v_cache) | page_bytes) & 15) return TS_ERR_UNSUPPORTED;
  const int pieces = (int)((page_bytes + PF_PIECE - 1) / PF_PIECE);
  const long long total = (long long)num_seqs * table_width * 2 * pieces;
  return launch(prefetch_pages_kernel, (unsigned int)((total + threads - 1) / threads), threads, 0, stream,
                (const char*)k_cache, (const char*)v_cache, page_bytes, block_tables, table_width, ctx_lens, num_seqs,
                page_size, pieces);
}

// Prefetch `count` (at most 8) ranges into L2. Every base must be 16-byte aligned; sizes are
// rounded down to a multiple of 16.
extern "C" int ts_prefetch_l2(const void* const* bases, const unsigned long long* sizes, int count, int threads,
                              cudaStream_t stream) {
  if (count <= 0) return 0;
  if (count > PF_MAX_RANGES || threads < 16 || threads > 128 || threads % 16 != 0) return TS_ERR_BAD_ARGUMENT;
  PrefetchRanges r;
  if (!prefetch_ranges_fill(&r, bases, sizes, count)) return TS_ERR_UNSUPPORTED;
  const unsigned int pieces = r.first_piece[PF_MAX_RANGES];
  if (pieces == 0) return 0;
  return launch(prefetch_l2_kernel, (pieces + threads - 1) / threads, threads, 0, stream, r);
}
