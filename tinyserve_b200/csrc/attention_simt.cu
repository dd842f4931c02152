// Entry point of the CUDA-core paged attention kernels (see attention_simt.cuh).
#define TS_PDL_CLASS PDL_ATTENTION
#include "attention_simt.cuh"

using namespace ts;

// Largest head_dim the SIMT kernels take: 16-element steps up to 256.
extern "C" int ts_attention_simt_max_head_dim() { return 256; }

extern "C" int ts_paged_attention_simt(
    const void* q, void* out, const void* k_cache, const void* v_cache, const int* block_tables,
    int table_width, const int* cu_q, const int* ctx_lens, const int* decode_seqs, int num_decode,
    const int* prefill_seqs, int num_prefill, int max_query_len, int num_heads, int num_kv_heads,
    int head_dim, int page_size, float scale, int window, int num_splits, float* part_acc,
    float* part_ml, int dtype, cudaStream_t stream) {
  if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 256) return TS_ERR_UNSUPPORTED;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || page_size <= 0 || window < 0) return TS_ERR_BAD_ARGUMENT;
  if (dtype != TS_DTYPE_F32 && dtype != TS_DTYPE_BF16) return TS_ERR_BAD_ARGUMENT;
  AttnArgs a;
  a.q = q; a.out = out; a.k_cache = k_cache; a.v_cache = v_cache;
  a.block_tables = block_tables; a.table_width = table_width; a.cu_q = cu_q; a.ctx_lens = ctx_lens;
  a.num_heads = num_heads; a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.page_size = page_size;
  a.page_shift = page_shift_of(page_size);
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  a.num_splits = 1; a.part_acc = nullptr; a.part_ml = nullptr;
  int st = 0;
  if (num_prefill > 0) {
    a.seq_ids = prefill_seqs; a.num_seqs = num_prefill;
    st = dtype == TS_DTYPE_F32 ? launch_prefill<float>(a, max_query_len, stream)
                               : launch_prefill<bf16>(a, max_query_len, stream);
    if (st != 0) return st;
  }
  if (num_decode > 0) {
    if (num_splits < 1 || num_splits > ATTN_MAX_SPLITS || (num_splits > 1 && (part_acc == nullptr || part_ml == nullptr))) return TS_ERR_BAD_ARGUMENT;
    a.seq_ids = decode_seqs; a.num_seqs = num_decode;
    a.num_splits = num_splits; a.part_acc = part_acc; a.part_ml = part_ml;
    st = dtype == TS_DTYPE_F32 ? launch_decode<float>(a, stream) : launch_decode<bf16>(a, stream);
  }
  return st;
}
