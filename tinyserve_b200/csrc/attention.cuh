// Arguments shared by the paged attention kernels.
#pragma once
#include "common.cuh"

namespace ts {

struct AttnArgs {
  const void* q;           // [T, num_heads, head_dim]
  void* out;               // [T, num_heads, head_dim]
  const void* k_cache;     // [pages, num_kv_heads, page_size, head_dim]
  const void* v_cache;
  const int* block_tables; // [B, table_width]
  const int* cu_q;         // [B + 1] first flat row of each request's new tokens
  const int* ctx_lens;     // [B] tokens of each request, the new ones included
  const int* seq_ids;      // requests this launch handles
  int num_seqs;            // how many of them
  int table_width;
  int num_heads, num_kv_heads, head_dim, page_size;
  int page_shift;          // log2(page_size) if it is a power of two, else -1
  float scale_log2;        // softmax scale times log2(e)
  int window;              // 0 = every earlier position; w = the last w positions
  // split-K decode
  int num_splits;
  float* part_acc;         // [num_seqs, num_heads, num_splits, head_dim]
  float* part_ml;          // [num_seqs, num_heads, num_splits, 2]  (max, sum)
};

__device__ __forceinline__ size_t kv_offset(int page, int kvh, int off, const AttnArgs& a) {
  return (((size_t)page * a.num_kv_heads + kvh) * a.page_size + off) * a.head_dim;
}

// Element offset of position `kpos` of a request (block table `table`) for kv head `kvh`.
__device__ __forceinline__ size_t kv_offset_of(const int* table, int kpos, int kvh, const AttnArgs& a) {
  int page, off;
  if (a.page_shift >= 0) {
    page = table[kpos >> a.page_shift];
    off = kpos & (a.page_size - 1);
  } else {
    const int idx = kpos / a.page_size;
    page = table[idx];
    off = kpos - idx * a.page_size;
  }
  return kv_offset(page, kvh, off, a);
}

static inline int page_shift_of(int page_size) {
  if (page_size <= 0 || (page_size & (page_size - 1))) return -1;
  int s = 0;
  while ((1 << s) < page_size) ++s;
  return s;
}

// Merge of the key ranges of one request for `ng` heads starting at `head0`, by a whole CTA:
// out = sum_s w_s acc_s / sum_s w_s l_s with w_s = 2^(m_s - max_s m_s). The (max, sum) pairs are
// staged in shared memory first (`ml` holds ng * S * 2 floats), so that the loop over the ranges
// issues independent loads.
template <typename T>
__device__ __forceinline__ void merge_splits(const AttnArgs& a, int si, int qrow, int head0, int ng, float* ml) {
  const int S = a.num_splits, D = a.head_dim;
  for (int idx = threadIdx.x; idx < ng * S * 2; idx += blockDim.x) {
    const int r = idx / (S * 2), rest = idx - r * (S * 2);
    ml[idx] = __ldcg(&a.part_ml[((size_t)si * a.num_heads + head0 + r) * S * 2 + rest]);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < ng * D; idx += blockDim.x) {
    const int r = idx / D, d = idx - r * D;
    const float* mlr = ml + (size_t)r * S * 2;
    float mm = -INFINITY;
    for (int sp = 0; sp < S; ++sp) mm = fmaxf(mm, mlr[sp * 2]);
    const float* acc = a.part_acc + ((size_t)si * a.num_heads + head0 + r) * S * D + d;
    float num = 0.f, den = 0.f;
    int sp = 0;
    for (; sp + 4 <= S; sp += 4) {
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldcg(acc + (size_t)(sp + u) * D);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float ms = mlr[(sp + u) * 2];
        const float c = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
        num += v[u] * c;
        den += mlr[(sp + u) * 2 + 1] * c;
      }
    }
    for (; sp < S; ++sp) {
      const float ms = mlr[sp * 2];
      const float c = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
      num += __ldcg(acc + (size_t)sp * D) * c;
      den += mlr[sp * 2 + 1] * c;
    }
    ((T*)a.out)[((size_t)qrow * a.num_heads + head0 + r) * D + d] = from_float<T>(num / den);
  }
}

constexpr int ATTN_MAX_SPLITS = 32;

}  // namespace ts
