// Ask the memory system to bring ranges of global memory into L2 ahead of their use
// (cp.async.bulk.prefetch.L2): a decode step reads every weight exactly once, one kernel after
// the other, and the attention kernel in the middle of a layer leaves part of the memory
// bandwidth idle; the weights that the products after it will stream are fetched meanwhile.
// The kernel only issues the requests (one thread per piece) and ends; nothing waits for the
// data, and nothing goes wrong if a line is evicted again before its use. No counterpart in
// upstream, whose products are library calls.
#include "common.cuh"

namespace ts {

constexpr int PF_MAX_RANGES = 8;
// Bytes per request; 128 threads per CTA. The kernel lasts until its requests are served, and an
// SM passes them on at about 0.15 TB/s, so the number of CTAs sets the rate: 16 KB x 128 threads
// fetches 23 MB with 12 CTAs at 1.9 TB/s in 11 us, about the length of the attention kernel it
// runs beside. Measured on B200 (Qwen3-0.6B sizes, batch 8): spread thinly over all SMs the same
// requests are served at 5.7 TB/s but take the bandwidth from the attention kernel (step 1.144 ms
// instead of 1.126 ms); slower than this, the step waits for the prefetch (1.27 ms). Fetching the
// next layer's cache pages the same way (beside the attention kernel, or beside the products
// after it) made every batch size slower, 1.33 ms at batch 8, and is not done.
constexpr unsigned int PF_PIECE = 16 * 1024;

struct PrefetchRanges {
  const char* base[PF_MAX_RANGES];
  unsigned long long bytes[PF_MAX_RANGES];        // multiples of 16
  unsigned int first_piece[PF_MAX_RANGES + 1];    // pieces before each range
  int count;
};

__global__ void prefetch_l2_kernel(PrefetchRanges r) {
  const unsigned int piece = blockIdx.x * blockDim.x + threadIdx.x;
  if (piece >= r.first_piece[r.count]) return;
  int i = 0;
  while (piece >= r.first_piece[i + 1]) ++i;
  const unsigned long long off = (unsigned long long)(piece - r.first_piece[i]) * PF_PIECE;
  const unsigned long long left = r.bytes[i] - off;
  const unsigned int n = left < PF_PIECE ? (unsigned int)left : PF_PIECE;
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(r.base[i] + off), "r"(n) : "memory");
}

}  // namespace ts

using namespace ts;

// Prefetch `count` (at most 8) ranges into L2. Every base must be 16-byte aligned; sizes are
// rounded down to a multiple of 16.
extern "C" int ts_prefetch_l2(const void* const* bases, const unsigned long long* sizes, int count, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (count > PF_MAX_RANGES) return TS_ERR_BAD_ARGUMENT;
  PrefetchRanges r;
  r.count = count;
  unsigned int pieces = 0;
  for (int i = 0; i < count; ++i) {
    if (((uintptr_t)bases[i]) & 15) return TS_ERR_UNSUPPORTED;
    r.base[i] = (const char*)bases[i];
    r.bytes[i] = sizes[i] & ~15ull;
    r.first_piece[i] = pieces;
    pieces += (unsigned int)((r.bytes[i] + PF_PIECE - 1) / PF_PIECE);
  }
  for (int i = count; i <= PF_MAX_RANGES; ++i) r.first_piece[i] = pieces;
  if (pieces == 0) return 0;
  return launch(prefetch_l2_kernel, (pieces + 127) / 128, 128, 0, stream, r);
}
