// Paged split-K decode attention on the tensor cores (bf16, head sizes 16..128 in steps of 16):
// one query token per request, all query heads of a kv group as the 16 rows of an mma tile.
// Math as in attention_simt.cuh (upstream src/tinyserve/attention.py:89-111; the split of a
// request's keys into ranges that are merged afterwards follows upstream
// src/tinyserve/triton_attention.py:243-327).
//
// The kernel is bound by the bytes of the cache it reads, so it is built to keep many of them in
// flight with few instructions: every warp runs its own two-stage pipeline of 16-key tiles; a
// tile is fetched by 32 bulk asynchronous copies (cp.async.bulk, one key row or value row per
// lane, completion counted by an mbarrier) into padded shared memory, read back with ldmatrix,
// and S = Q K^T and O += P V are mma.sync m16n8k16 with 32-bit accumulators; the softmax is
// online, 32-bit, base 2. A CTA is one (request, kv group, key range); its four warps take
// tiles in turn and merge at the end; the CTA that finishes a request's last range merges the
// ranges (arrival counter), so there is no second kernel.
// Every mbarrier wait is bounded; a wait that runs out sets *error_flag and the CTA leaves.
#define TS_PDL_CLASS PDL_ATTENTION
#include "attention.cuh"
#include "bounded_wait.cuh"

namespace ts {

#ifndef DM_STAGES_N
#define DM_STAGES_N 2
#endif
constexpr int DM_WARPS = 4, DM_THREADS = DM_WARPS * 32, DM_TK = 16, DM_STAGES = DM_STAGES_N;
constexpr int DM_MAX_COUNTERS = 1 << 16;

static __device__ unsigned int g_dm_arrivals[DM_MAX_COUNTERS];

__device__ __forceinline__ uint32_t dm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void dm_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(dm_smem(p)));
}
__device__ __forceinline__ void dm_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(dm_smem(p)));
}
__device__ __forceinline__ void dm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t dm_pack(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void dm_bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(dm_smem(bar)), "r"(count));
}
__device__ __forceinline__ void dm_bar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(dm_smem(bar)) : "memory");
}
__device__ __forceinline__ void dm_bar_arrive_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(dm_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool dm_bar_wait(uint64_t* bar, uint32_t parity) {
  return bounded_mbar_wait(dm_smem(bar), parity);
}
// One row of the cache (bytes a multiple of 16, both addresses 16-byte aligned) -> shared memory.
__device__ __forceinline__ void dm_bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dm_smem(dst)), "l"(src), "r"(bytes), "r"(dm_smem(bar)) : "memory");
}

// D16 = head_dim / 16. blockIdx = (request in the list, kv head * passes + pass, key range).
// A pass covers up to 16 query heads of the group.
template <int D16>
__global__ void __launch_bounds__(DM_THREADS) decode_attn_mma_kernel(AttnArgs a, int passes, int* error_flag) {
  constexpr int D = D16 * 16, DS = D + 8;
  constexpr int TILE_ELEMS = DM_TK * DS;                    // one K (or V) tile of a stage
  extern __shared__ __align__(16) unsigned char dm_raw[];
  __shared__ __align__(8) uint64_t bars[DM_WARPS][DM_STAGES];
  __shared__ int is_last;
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  bf16* my_k = reinterpret_cast<bf16*>(dm_raw) + (size_t)warp * DM_STAGES * 2 * TILE_ELEMS;   // [stage][K|V][32][DS]
  const int G = a.num_heads / a.num_kv_heads;
  const int si = blockIdx.x;
  const int kvh = blockIdx.y / passes;
  const int g0 = (blockIdx.y - kvh * passes) * 16;
  const int ng = min(16, G - g0);
  const int split = blockIdx.z;
  if (lane == 0) {
    for (int s = 0; s < DM_STAGES; ++s) dm_bar_init(&bars[warp][s], 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  pdl_wait();

  const int seq = a.seq_ids[si];
  const int ctx = a.ctx_lens[seq];
  const int qrow = a.cu_q[seq];
  const int lo = (a.window > 0) ? max(0, ctx - a.window) : 0;
  const int lo_al = lo & ~(DM_TK - 1);
  const int ntiles_all = (ctx - lo_al + DM_TK - 1) / DM_TK;
  const int tiles_per = (ntiles_all + a.num_splits - 1) / a.num_splits;
  const int tile_begin = split * tiles_per;
  const int tile_end = min(ntiles_all, tile_begin + tiles_per);
  const int* table = a.block_tables + (size_t)seq * a.table_width;
  const bf16* kc = (const bf16*)a.k_cache;
  const bf16* vc = (const bf16*)a.v_cache;

  // ---- Q fragments: row r = query head g0 + r of the group (rows beyond the group are zero)
  uint32_t qf[D16][4];
  {
    const bf16* qbase = (const bf16*)a.q + ((size_t)qrow * a.num_heads + kvh * G + g0) * D;
#pragma unroll
    for (int kk = 0; kk < D16; ++kk) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = g + 8 * h;
        uint32_t lo_w = 0u, hi_w = 0u;
        if (r < ng) {
          lo_w = *reinterpret_cast<const uint32_t*>(qbase + (size_t)r * D + kk * 16 + 2 * t);
          hi_w = *reinterpret_cast<const uint32_t*>(qbase + (size_t)r * D + kk * 16 + 8 + 2 * t);
        }
        qf[kk][h] = lo_w;
        qf[kk][2 + h] = hi_w;
      }
    }
  }

  auto load_tile = [&](int tile, int stage) {
    // lanes 0-15 fetch the 16 key rows of the tile, lanes 16-31 its value rows (or zero them
    // if the position lies outside the request's range)
    if (wait_test_unarmed()) return;
    const int row = lane & 15;
    const int kpos = lo_al + tile * DM_TK + row;
    bf16* dst = my_k + (size_t)stage * 2 * TILE_ELEMS + (lane >> 4) * TILE_ELEMS + row * DS;
    if (kpos >= lo && kpos < ctx) {
      const size_t off = kv_offset_of(table, kpos, kvh, a);
      dm_bar_arrive_tx(&bars[warp][stage], D * 2u);
      dm_bulk_copy(dst, ((lane >> 4) ? vc : kc) + off, D * 2u, &bars[warp][stage]);
    } else {
#pragma unroll
      for (int c = 0; c < D / 8; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0u, 0u, 0u, 0u);
      dm_bar_arrive(&bars[warp][stage]);
    }
  };

  float o[2 * D16][4];
#pragma unroll
  for (int i = 0; i < 2 * D16; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  bool failed = false;

  // this warp's tiles: tile_begin + warp, + DM_WARPS, ...
  const int first = tile_begin + warp;
  int issued = 0;
  for (int s = 0; s < DM_STAGES; ++s) {
    const int tile = first + s * DM_WARPS;
    if (tile < tile_end) { load_tile(tile, s); ++issued; }
  }
  int n = 0;
  for (int tile = first; tile < tile_end; tile += DM_WARPS, ++n) {
    const int stage = n % DM_STAGES;
    const uint32_t parity = (n / DM_STAGES) & 1;
    if (!dm_bar_wait(&bars[warp][stage], parity)) { failed = true; break; }
    __syncwarp();
    const bf16* kt = my_k + (size_t)stage * 2 * TILE_ELEMS;
    const bf16* vt = kt + TILE_ELEMS;
    const int k0 = lo_al + tile * DM_TK;
    // ---- S = Q K^T: 2 key tiles of 8
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D16; ++kk) {
      uint32_t bfr[4];
      const int key = (lane & 7) + (lane >> 4) * 8;
      const int c = kk * 16 + ((lane >> 3) & 1) * 8;
      dm_ldmatrix_x4(bfr, kt + key * DS + c);
      dm_mma(s[0], qf[kk], bfr[0], bfr[1]);
      dm_mma(s[1], qf[kk], bfr[2], bfr[3]);
    }
    // ---- scale, mask (keys outside [lo, ctx)), online softmax for rows g and g + 8
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kpos = k0 + i * 8 + 2 * t + (e & 1);
        const bool ok = kpos >= lo && kpos < ctx;
        const float v = ok ? s[i][e] * a.scale_log2 : -INFINITY;
        s[i][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m[h], mx[h]);
      corr[h] = (m_new == -INFINITY) ? 1.f : exp2f(m[h] - m_new);
      m[h] = m_new;
      l[h] *= corr[h];
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = (s[i][e] == -INFINITY) ? 0.f : exp2f(s[i][e] - m[e >> 1]);
        s[i][e] = p;
        l[e >> 1] += p;
      }
#pragma unroll
    for (int i = 0; i < 2 * D16; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0];
      o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    // ---- O += P V: one step of 16 keys
    {
      uint32_t pf[4];
      pf[0] = dm_pack(s[0][0], s[0][1]);
      pf[1] = dm_pack(s[0][2], s[0][3]);
      pf[2] = dm_pack(s[1][0], s[1][1]);
      pf[3] = dm_pack(s[1][2], s[1][3]);
#pragma unroll
      for (int dp = 0; dp < D16; ++dp) {
        uint32_t vfr[4];
        const int key = (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = dp * 16 + (lane >> 4) * 8;
        dm_ldmatrix_x4_trans(vfr, vt + key * DS + c);
        dm_mma(o[2 * dp], pf, vfr[0], vfr[1]);
        dm_mma(o[2 * dp + 1], pf, vfr[2], vfr[3]);
      }
    }
    __syncwarp();                                  // every lane is done with this stage
    const int nxt = tile + DM_STAGES * DM_WARPS;
    if (nxt < tile_end) load_tile(nxt, stage);
  }
  if (failed && lane == 0) atomicExch(error_flag, WAIT_FAILED_DECODE_BULK);

  // ---- row sums across the quad; then merge the warps through shared memory
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  __syncthreads();                                 // all warps are done with their tiles
  float* red = reinterpret_cast<float*>(dm_raw);   // [DM_WARPS][16][D + 2], reusing the tile memory
  constexpr int WS = D + 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + 8 * h;
    if (r < ng) {
      float* w = red + ((size_t)warp * 16 + r) * WS;
#pragma unroll
      for (int i = 0; i < 2 * D16; ++i) {
        w[i * 8 + 2 * t] = o[i][2 * h];
        w[i * 8 + 2 * t + 1] = o[i][2 * h + 1];
      }
      if (t == 0) { w[D] = m[h]; w[D + 1] = l[h]; }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < ng * D; idx += DM_THREADS) {
    const int r = idx / D, d = idx - r * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) mm = fmaxf(mm, red[((size_t)w * 16 + r) * WS + D]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) {
      const float* ws = red + ((size_t)w * 16 + r) * WS;
      const float c = (ws[D] == -INFINITY) ? 0.f : exp2f(ws[D] - mm);
      num += ws[d] * c;
      den += ws[D + 1] * c;
    }
    const int head = kvh * G + g0 + r;
    if (a.num_splits == 1) {
      ((bf16*)a.out)[((size_t)qrow * a.num_heads + head) * D + d] = __float2bfloat16_rn(num / den);
    } else {
      const size_t pidx = ((size_t)si * a.num_heads + head) * a.num_splits + split;
      a.part_acc[pidx * D + d] = num;
      if (d == 0) { a.part_ml[pidx * 2] = mm; a.part_ml[pidx * 2 + 1] = den; }
    }
  }
  if (a.num_splits == 1) return;
  // ---- the CTA that arrives last for this (request, heads) merges the ranges
  unsigned int* counter = &g_dm_arrivals[((size_t)si * gridDim.y + blockIdx.y) % DM_MAX_COUNTERS];
  if (!cta_arrives_last(counter, (unsigned int)a.num_splits, &is_last)) return;
  merge_splits<bf16>(a, si, qrow, kvh * G + g0, ng, red);
}

template <int D16>
static int launch_dm(const AttnArgs& a, int* error_flag, cudaStream_t stream) {
  constexpr int DS = D16 * 16 + 8;
  const size_t tiles = sizeof(bf16) * (size_t)DM_WARPS * DM_STAGES * 2 * DM_TK * DS;
  const size_t red = sizeof(float) * (size_t)DM_WARPS * 16 * (D16 * 16 + 2);
  const size_t smem = tiles > red ? tiles : red;
  auto kern = decode_attn_mma_kernel<D16>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int G = a.num_heads / a.num_kv_heads;
  const int passes = (G + 15) / 16;
  if (a.num_splits > 1 && (long long)a.num_seqs * a.num_kv_heads * passes > DM_MAX_COUNTERS) return TS_ERR_UNSUPPORTED;
  dim3 grid(a.num_seqs, a.num_kv_heads * passes, a.num_splits);
  return launch(kern, grid, DM_THREADS, smem, stream, a, passes, error_flag);
}

}  // namespace ts

using namespace ts;

// bf16 decode attention for the requests listed in decode_seqs (one token each).
// head_dim in {16, ..., 128}; part_acc / part_ml as in ts_paged_attention_simt when num_splits > 1.
extern "C" int ts_decode_attention_mma(
    const void* q, void* out, const void* k_cache, const void* v_cache, const int* block_tables,
    int table_width, const int* cu_q, const int* ctx_lens, const int* decode_seqs, int num_decode,
    int num_heads, int num_kv_heads, int head_dim, int page_size, float scale, int window, int num_splits,
    float* part_acc, float* part_ml, int* error_flag, cudaStream_t stream) {
  if (num_decode <= 0) return 0;
  if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 128 || error_flag == nullptr) return TS_ERR_UNSUPPORTED;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || page_size <= 0 || window < 0 || num_splits < 1 || num_splits > ATTN_MAX_SPLITS)
    return TS_ERR_BAD_ARGUMENT;
  if (num_splits > 1 && (part_acc == nullptr || part_ml == nullptr)) return TS_ERR_BAD_ARGUMENT;
  if ((((uintptr_t)k_cache) | ((uintptr_t)v_cache)) & 15) return TS_ERR_UNSUPPORTED;
  AttnArgs a;
  a.q = q; a.out = out; a.k_cache = k_cache; a.v_cache = v_cache;
  a.block_tables = block_tables; a.table_width = table_width; a.cu_q = cu_q; a.ctx_lens = ctx_lens;
  a.seq_ids = decode_seqs; a.num_seqs = num_decode;
  a.num_heads = num_heads; a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.page_size = page_size;
  a.page_shift = page_shift_of(page_size);
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  a.num_splits = num_splits; a.part_acc = part_acc; a.part_ml = part_ml;
  switch (head_dim / 16) {
    case 1: return launch_dm<1>(a, error_flag, stream);
    case 2: return launch_dm<2>(a, error_flag, stream);
    case 3: return launch_dm<3>(a, error_flag, stream);
    case 4: return launch_dm<4>(a, error_flag, stream);
    case 5: return launch_dm<5>(a, error_flag, stream);
    case 6: return launch_dm<6>(a, error_flag, stream);
    case 7: return launch_dm<7>(a, error_flag, stream);
    case 8: return launch_dm<8>(a, error_flag, stream);
  }
  return TS_ERR_UNSUPPORTED;
}

// How many CTAs of the tensor-core decode kernel fit the machine at once (for the split choice).
extern "C" int ts_decode_attention_mma_slots(int head_dim) {
  const int ds = head_dim + 8;
  const size_t smem = sizeof(bf16) * (size_t)DM_WARPS * DM_STAGES * 2 * DM_TK * ds + 1024;
  int per_sm = (int)((227 * 1024) / smem);
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 8) per_sm = 8;
  return 148 * per_sm;
}
