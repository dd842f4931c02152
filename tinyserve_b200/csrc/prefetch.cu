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

}  // namespace ts

using namespace ts;

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
