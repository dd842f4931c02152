// Paged split-K decode attention with its scratch in a fixed device array of the library:
// an entry point for callers that may not allocate (see decode_attention_static_scratch.h,
// which states the limits). The kernels are the ones of attention_simt.cuh; only where the
// partial results live differs from ts_paged_attention_simt.
#define TS_PDL_CLASS PDL_ATTENTION
#include "decode_attention_static_scratch.h"

#include "attention_simt.cuh"

static_assert(TS_STATIC_SCRATCH_MAX_SPLITS == ts::ATTN_MAX_SPLITS, "the header states the launchers' limit");

namespace {

// Partial (max, sum, accumulator) of every key range. In host code this name is only a
// handle for cudaGetSymbolAddress; its device address is looked up once per device below.
static __device__ __align__(256) float g_static_scratch[TS_STATIC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_scratch_ptr[MAX_DEVICES] = {};

// Device address of the scratch array on the current device (looked up on first use).
int scratch_address(float** ptr) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return TS_ERR_UNSUPPORTED;
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return TS_ERR_UNSUPPORTED;
    g_scratch_ptr[dev] = p;
  }
  *ptr = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" long long ts_decode_attention_static_scratch_need(int num_decode, int num_heads, int head_dim,
                                                             int num_splits) {
  if (num_splits <= 1) return 0;
  return (long long)num_decode * num_heads * num_splits * ((long long)head_dim + 2);
}

extern "C" int ts_decode_attention_static_scratch(const void* q, void* out, const void* k_cache,
                                                  const void* v_cache, const int* block_tables, int table_width,
                                                  const int* cu_q, const int* ctx_lens, const int* decode_seqs,
                                                  int num_decode, int num_heads, int num_kv_heads, int head_dim,
                                                  int page_size, float scale, int window, int num_splits,
                                                  int dtype, cudaStream_t stream) {
  using namespace ts;
  if (num_decode <= 0) return 0;
  if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 256) return TS_ERR_UNSUPPORTED;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || page_size <= 0 || window < 0 || num_splits < 1 || num_splits > ATTN_MAX_SPLITS)
    return TS_ERR_BAD_ARGUMENT;
  if (dtype != TS_DTYPE_F32 && dtype != TS_DTYPE_BF16) return TS_ERR_BAD_ARGUMENT;
  const long long need = ts_decode_attention_static_scratch_need(num_decode, num_heads, head_dim, num_splits);
  if (need > (long long)TS_STATIC_SCRATCH_FLOATS) return TS_ERR_SCRATCH_TOO_SMALL;

  AttnArgs a;
  a.q = q; a.out = out; a.k_cache = k_cache; a.v_cache = v_cache;
  a.block_tables = block_tables; a.table_width = table_width; a.cu_q = cu_q; a.ctx_lens = ctx_lens;
  a.seq_ids = decode_seqs; a.num_seqs = num_decode;
  a.num_heads = num_heads; a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.page_size = page_size;
  a.page_shift = page_shift_of(page_size);
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  a.num_splits = num_splits; a.part_acc = nullptr; a.part_ml = nullptr;
  if (num_splits > 1) {
    float* scratch = nullptr;
    const int st = scratch_address(&scratch);
    if (st != 0) return st;
    // accumulators first, then the (max, sum) pairs; both offsets keep 8-byte alignment
    a.part_acc = scratch;
    a.part_ml = scratch + (long long)num_decode * num_heads * num_splits * head_dim;
  }
  return dtype == TS_DTYPE_F32 ? launch_decode<float>(a, stream) : launch_decode<bf16>(a, stream);
}
