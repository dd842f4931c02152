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

}  // namespace ts
