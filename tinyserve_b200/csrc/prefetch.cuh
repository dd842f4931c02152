// A list of global-memory ranges to be brought into L2 (cp.async.bulk.prefetch.L2), cut into pieces
// of 16 KB that any thread of any kernel can ask for (the prefetch kernel of prefetch.cu walks it).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ts {

constexpr int PF_MAX_RANGES = 8;
constexpr unsigned int PF_PIECE = 16 * 1024;

struct PrefetchRanges {
  const char* base[PF_MAX_RANGES];
  unsigned long long bytes[PF_MAX_RANGES];        // multiples of 16
  unsigned int first_piece[PF_MAX_RANGES + 1];    // pieces before each range
  int count;                                      // 0: nothing to fetch
};

__device__ __forceinline__ void prefetch_piece(const PrefetchRanges& r, unsigned int piece) {
  if (piece >= r.first_piece[r.count]) return;
  int i = 0;
  while (piece >= r.first_piece[i + 1]) ++i;
  const unsigned long long off = (unsigned long long)(piece - r.first_piece[i]) * PF_PIECE;
  const unsigned long long left = r.bytes[i] - off;
  const unsigned int n = left < PF_PIECE ? (unsigned int)left : PF_PIECE;
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(r.base[i] + off), "r"(n) : "memory");
}

// Host side: fill `r` from `count` ranges (every base 16-byte aligned; sizes are rounded down to a
// multiple of 16). Returns false if a base is misaligned or there are too many ranges.
static inline bool prefetch_ranges_fill(PrefetchRanges* r, const void* const* bases, const unsigned long long* sizes,
                                        int count) {
  r->count = 0;
  for (int i = 0; i <= PF_MAX_RANGES; ++i) r->first_piece[i] = 0;
  if (count <= 0) return true;
  if (count > PF_MAX_RANGES) return false;
  unsigned int pieces = 0;
  for (int i = 0; i < count; ++i) {
    if (((uintptr_t)bases[i]) & 15) return false;
    r->base[i] = (const char*)bases[i];
    r->bytes[i] = sizes[i] & ~15ull;
    r->first_piece[i] = pieces;
    pieces += (unsigned int)((r->bytes[i] + PF_PIECE - 1) / PF_PIECE);
  }
  for (int i = count; i <= PF_MAX_RANGES; ++i) r->first_piece[i] = pieces;
  r->count = pieces ? count : 0;
  return true;
}

}  // namespace ts
