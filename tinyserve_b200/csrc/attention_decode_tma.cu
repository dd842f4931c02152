// Paged split-K decode attention on the tensor cores with TMA tile loads (bf16, head sizes 64 and
// 128, page sizes 8 or a multiple of 16): the variant of attention_decode_mma.cu that fetches a
// 16-key tile with a few tensor copies instead of one bulk copy per row.
// one query token per request, all query heads of a kv group as the 16 rows of an mma tile.
// Math as in attention_simt.cuh (upstream src/tinyserve/attention.py:89-111; the split of a
// request's keys into ranges that are merged afterwards follows upstream
// src/tinyserve/triton_attention.py:243-327).
//
// The cache of one layer is described to the TMA unit as a matrix of (page, kv head, offset) rows
// by head_dim columns. A tile is 16 consecutive positions of one kv head, which lie in one page
// (or two pages of 8): one lane fetches it with cp.async.bulk.tensor boxes of 16 (or 8) rows by
// 64 columns, 128-byte swizzled, completion counted by an mbarrier; ldmatrix reads the swizzled
// rows without bank conflicts and without padding. Rows of a tile that lie outside the request's
// range hold whatever the page holds there; their scores are masked and their values zeroed
// before use. Every warp runs its own two-stage pipeline of tiles;
// S = Q K^T and O += P V are mma.sync m16n8k16 with 32-bit accumulators; the softmax is
// online, 32-bit, base 2. A CTA is one (request, kv group, key range); its four warps take
// tiles in turn and merge at the end; the CTA that finishes a request's last range merges the
// ranges (arrival counter), so there is no second kernel.
// Every mbarrier wait is bounded; a wait that runs out sets *error_flag and the CTA leaves.
#define TS_PDL_CLASS PDL_ATTENTION
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "attention.cuh"
#include "bounded_wait.cuh"

namespace ts {

#ifndef DM_STAGES_N
#define DM_STAGES_N 2
#endif
constexpr int DM_WARPS = 4, DM_THREADS = DM_WARPS * 32, DM_TK = 16, DM_STAGES = DM_STAGES_N;
constexpr int DM_MAX_COUNTERS = 1 << 16;

static __device__ unsigned int g_dt_arrivals[DM_MAX_COUNTERS];

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
// A box of rows x 64 columns of the cache matrix -> shared memory, 128-byte swizzled.
__device__ __forceinline__ void dm_tensor_copy(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dm_smem(dst)), "l"(map), "r"(dm_smem(bar)), "r"(x), "r"(y) : "memory");
}
// Address of the 16-byte chunk `chunk` (of head_dim / 8) of row `row` (0..15) of a swizzled tile:
// sub-tiles of 64 columns are 2 KiB apart; within one, a row is 128 bytes and its chunks are
// permuted by the row's low three bits.
__device__ __forceinline__ const unsigned char* dm_swizzled(const unsigned char* tile, int row, int chunk) {
  return tile + (chunk >> 3) * 2048 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

// What the fused variant needs besides the attention arguments: the raw output of the qkv
// product and what turns it into queries, keys and values (per-head RMSNorm weights, rotary
// tables, cache slots). With it the kernel does the work of qk_rope_write.cu itself: every CTA
// normalises and rotates its own query heads; the CTA that owns a request's last key range also
// normalises, rotates and stores the new key and value, and patches them into its tile.
struct FusedQkv {
  const bf16* qkv;         // [tokens, (num_heads + 2 num_kv_heads) * head_dim]
  const bf16* q_weight;    // [head_dim] or null (no norm)
  const bf16* k_weight;
  float eps;
  const float* cos_t;      // [tokens, head_dim / 2] or null (no rotation)
  const float* sin_t;
  const int* slots;        // [tokens] cache slot of each new token
  bf16* k_cache;           // writable views of the cache
  bf16* v_cache;
};

// One head row (head_dim elements at src): optional RMSNorm with weight, optional rotate-half
// rotation with the token's tables; result rounded to bf16 into dst0 and, if given, dst1.
// Executed by a whole warp. Rounding points as in qk_rope_write.cu.
// A lane's share of a per-head norm weight (the elements fused_head_row gives it). The weights
// are constants of the model, so they are loaded before the kernel waits for its predecessor.
template <int D>
struct HeadWeight {
  static constexpr int MAXJ = (D / 2 + 63) / 64;
  uint32_t a[MAXJ], b[MAXJ];
  bool given;
  __device__ __forceinline__ void load(const bf16* weight, int lane) {
    given = weight != nullptr;
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int p = 2 * lane + 64 * j;
      a[j] = b[j] = 0x3f803f80u;                 // bf16 ones
      if (given && p < D / 2) {
        a[j] = *reinterpret_cast<const uint32_t*>(weight + p);
        b[j] = *reinterpret_cast<const uint32_t*>(weight + D / 2 + p);
      }
    }
  }
};

template <int D>
__device__ __forceinline__ void fused_head_row(const bf16* src, const HeadWeight<D>& weight, float eps, const float* c,
                                               const float* s, bf16* dst0, bf16* dst1, int lane) {
  constexpr int HALF = D / 2, MAXJ = (HALF + 63) / 64;
  // every load first (row, tables), so that they travel together
  uint32_t xa[MAXJ], xb[MAXJ];
  float2 cv[MAXJ], sv[MAXJ];
#pragma unroll
  for (int j = 0; j < MAXJ; ++j) {
    const int p = 2 * lane + 64 * j;
    xa[j] = xb[j] = 0u;
    cv[j] = make_float2(1.f, 1.f);
    sv[j] = make_float2(0.f, 0.f);
    if (p < HALF) {
      xa[j] = *reinterpret_cast<const uint32_t*>(src + p);
      xb[j] = *reinterpret_cast<const uint32_t*>(src + HALF + p);
      if (c != nullptr) {
        cv[j] = *reinterpret_cast<const float2*>(c + p);
        sv[j] = *reinterpret_cast<const float2*>(s + p);
      }
    }
  }
  float a[MAXJ][2], b[MAXJ][2];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXJ; ++j) {
    a[j][0] = __uint_as_float(xa[j] << 16); a[j][1] = __uint_as_float(xa[j] & 0xffff0000u);
    b[j][0] = __uint_as_float(xb[j] << 16); b[j][1] = __uint_as_float(xb[j] & 0xffff0000u);
    ss += a[j][0] * a[j][0] + a[j][1] * a[j][1] + b[j][0] * b[j][0] + b[j][1] * b[j][1];
  }
  if (weight.given) {
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + eps);
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const float fa[2] = {__uint_as_float(weight.a[j] << 16), __uint_as_float(weight.a[j] & 0xffff0000u)};
      const float fb[2] = {__uint_as_float(weight.b[j] << 16), __uint_as_float(weight.b[j] & 0xffff0000u)};
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        a[j][e] = round_to<bf16>(round_to<bf16>(a[j][e] * rstd) * fa[e]);
        b[j][e] = round_to<bf16>(round_to<bf16>(b[j][e] * rstd) * fb[e]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < MAXJ; ++j) {
    const int p = 2 * lane + 64 * j;
    if (p < HALF) {
      float ra[2] = {a[j][0], a[j][1]}, rb[2] = {b[j][0], b[j][1]};
      if (c != nullptr) {
        ra[0] = a[j][0] * cv[j].x - b[j][0] * sv[j].x; ra[1] = a[j][1] * cv[j].y - b[j][1] * sv[j].y;
        rb[0] = b[j][0] * cv[j].x + a[j][0] * sv[j].x; rb[1] = b[j][1] * cv[j].y + a[j][1] * sv[j].y;
      }
      const uint32_t pa = dm_pack(ra[0], ra[1]), pb = dm_pack(rb[0], rb[1]);
      *reinterpret_cast<uint32_t*>(dst0 + p) = pa;
      *reinterpret_cast<uint32_t*>(dst0 + HALF + p) = pb;
      if (dst1 != nullptr) {
        *reinterpret_cast<uint32_t*>(dst1 + p) = pa;
        *reinterpret_cast<uint32_t*>(dst1 + HALF + p) = pb;
      }
    }
  }
}

// D64 = head_dim / 64 (1 or 2). BR = rows of a tensor box: 16 (page size a multiple of 16) or 8.
// blockIdx = (request in the list, kv head * passes + pass, key range); a pass covers up to 16
// query heads of the group.
// WARPS: warps per CTA (4; 3 where one more CTA per SM lets a grid run as a single wave).
// CLUSTER: the CTAs of the key ranges of one (request, kv head, pass) form a thread-block cluster
// (1, 1, num_splits) and merge their results through distributed shared memory instead of through
// global memory and an arrival counter: the tail of the kernel, where no key is in flight any
// more, is two cluster barriers long instead of two trips to L2 and one atomic.
template <int D64, int BR, bool FUSED, int WARPS, bool CLUSTER>
__global__ void __launch_bounds__(WARPS * 32) decode_attn_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                     const __grid_constant__ CUtensorMap map_v,
                                                                     AttnArgs a, FusedQkv f, int passes,
                                                                     int* error_flag) {
  constexpr int D = D64 * 64, D16 = D / 16;
  constexpr int TILE_BYTES = DM_TK * D * 2;                 // one K (or V) tile: 16 rows, unpadded
  extern __shared__ __align__(16) unsigned char dm_raw[];
  __shared__ __align__(8) uint64_t bars[WARPS][DM_STAGES];
  __shared__ int is_last;
  // (CLUSTER) what the other ranges' CTAs send this CTA for the outputs it merges: their sums for its
  // share of the ng x D outputs, and every row's maximum and weight
  constexpr int RECV_CAP = 640;
  __shared__ float recv_num[CLUSTER ? RECV_CAP : 1];
  __shared__ float recv_ml[CLUSTER ? 8 * 16 * 2 : 1];
  // this CTA's query heads, ready for the mma. Rows are 8 elements (16 bytes) further apart than a
  // head is long: the fragment loads below read rows g = 0..7 at the same column, and rows that are
  // a multiple of 128 bytes apart would all fall into the same banks (an 8-way conflict on each of
  // the 32 loads of a warp: 320 k conflicts in a launch of 320 CTAs)
  constexpr int QS = FUSED ? D + 8 : D;
  __shared__ __align__(16) bf16 q_stage[FUSED ? 16 * (128 + 8) : 8];
  __shared__ __align__(16) bf16 new_kv[FUSED ? 2 * 128 : 8];       // the new token's key and value rows
  pdl_trigger();
  unsigned char* tiles = (unsigned char*)(((uintptr_t)dm_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  unsigned char* my = tiles + (size_t)warp * DM_STAGES * 2 * TILE_BYTES;      // [stage][K|V][tile]
  const int G = a.num_heads / a.num_kv_heads;
  const int si = blockIdx.x;
  const int kvh = blockIdx.y / passes;
  const int g0 = (blockIdx.y - kvh * passes) * 16;
  const int ng = min(16, G - g0);
  const int split = blockIdx.z;
  if (lane == 0) {
    for (int s = 0; s < DM_STAGES; ++s) dm_bar_init(&bars[warp][s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  // Nothing that the kernels just before this one write is read until the first tiles are on
  // their way: lengths and block tables are the step's host-made inputs, and the cache rows of
  // earlier positions were written in earlier steps. Only the tile with the newest position
  // (written by the kernel before, or, in the fused form, taken from shared memory) and the
  // queries wait for the predecessor.

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

  // One lane fetches a tile: the 16 positions from k0 lie in one page (BR = 16) or in two pages
  // of 8. Row of the cache matrix = (page * kv_heads + kvh) * page_size + offset in the page.
  auto load_tile = [&](int tile, int stage) {
    if (lane != 0 || wait_test_unarmed()) return;
    const int k0 = lo_al + tile * DM_TK;
    unsigned char* kd = my + (size_t)stage * 2 * TILE_BYTES;
    unsigned char* vd = kd + TILE_BYTES;
    uint64_t* bar = &bars[warp][stage];
    dm_bar_arrive_tx(bar, 2u * TILE_BYTES);
#pragma unroll
    for (int part = 0; part < DM_TK / BR; ++part) {
      int kpos = k0 + part * BR;
      if (kpos >= ctx) kpos = k0;      // a part wholly past the end: fetch any valid rows, they are masked
      int page, off;
      if (a.page_shift >= 0) { page = table[kpos >> a.page_shift]; off = kpos & (a.page_size - 1); }
      else { const int idx = kpos / a.page_size; page = table[idx]; off = kpos - idx * a.page_size; }
      const int y = (page * a.num_kv_heads + kvh) * a.page_size + off;
#pragma unroll
      for (int h = 0; h < D64; ++h) {
        dm_tensor_copy(kd + h * 2048 + part * BR * 128, &map_k, h * 64, y, bar);
        dm_tensor_copy(vd + h * 2048 + part * BR * 128, &map_v, h * 64, y, bar);
      }
    }
  };

  float o[2 * D16][4];
#pragma unroll
  for (int i = 0; i < 2 * D16; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  bool failed = false;

  // this warp's tiles: tile_begin + warp, + WARPS, ...
  const int first = tile_begin + warp;
  for (int s = 0; s < DM_STAGES; ++s) {
    const int tile = first + s * WARPS;
    if (tile < tile_end && (FUSED || tile < ntiles_all - 1)) load_tile(tile, s);
  }
  // (fused form) constants of the model and host-made inputs of the step, before the wait too
  const bool owns_last = tile_begin < tile_end && tile_end == ntiles_all;   // this range ends at the newest key
  HeadWeight<D> q_w, k_w;
  int new_slot = 0;
  if constexpr (FUSED) {
    q_w.load(f.q_weight, lane);
    if (owns_last) {
      k_w.load(f.k_weight, lane);
      new_slot = f.slots[qrow];
    }
  }
  pdl_wait();
  if constexpr (!FUSED) {
    for (int s = 0; s < DM_STAGES; ++s) {
      const int tile = first + s * WARPS;
      if (tile < tile_end && tile == ntiles_all - 1) load_tile(tile, s);
    }
  }

  // (the first tiles are on their way; the work on the queries overlaps their flight)
  if constexpr (FUSED) {
    const int width = (a.num_heads + 2 * a.num_kv_heads) * D;
    const bf16* row = f.qkv + (size_t)qrow * width;
    const float* c = f.cos_t ? f.cos_t + (size_t)qrow * (D / 2) : nullptr;
    const float* sn = f.sin_t ? f.sin_t + (size_t)qrow * (D / 2) : nullptr;
    for (int r = warp; r < 16; r += WARPS) {
      if (r < ng) {
        fused_head_row<D>(row + (size_t)(kvh * G + g0 + r) * D, q_w, f.eps, c, sn, q_stage + r * QS, nullptr, lane);
      } else {
        for (int i = lane * 8; i < D; i += 256) *reinterpret_cast<uint4*>(q_stage + r * QS + i) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    if (owns_last) {
      // the new key (normalised, rotated) and value: into the cache for later steps (once per
      // kv head: the CTA of the first pass writes) and into shared memory for this step
      const int page = new_slot / a.page_size, off = new_slot - page * a.page_size;
      const size_t at = kv_offset(page, kvh, off, a);
      const bool writer = (g0 == 0);
      if (warp == (ng % WARPS)) {
        fused_head_row<D>(row + (size_t)(a.num_heads + kvh) * D, k_w, f.eps, c, sn, new_kv,
                          writer ? f.k_cache + at : nullptr, lane);
      } else if (warp == ((ng + 1) % WARPS)) {
        const bf16* vsrc = row + (size_t)(a.num_heads + a.num_kv_heads + kvh) * D;
        for (int i = lane * 8; i < D; i += 256) {
          const uint4 v = *reinterpret_cast<const uint4*>(vsrc + i);
          *reinterpret_cast<uint4*>(new_kv + D + i) = v;
          if (writer) *reinterpret_cast<uint4*>(f.v_cache + at + i) = v;
        }
      }
    }
    __syncthreads();
  }

  // ---- Q fragments: row r = query head g0 + r of the group (rows beyond the group are zero)
  uint32_t qf[D16][4];
  {
    const bf16* qbase = FUSED ? q_stage : (const bf16*)a.q + ((size_t)qrow * a.num_heads + kvh * G + g0) * D;
#pragma unroll
    for (int kk = 0; kk < D16; ++kk) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = g + 8 * h;
        uint32_t lo_w = 0u, hi_w = 0u;
        if (FUSED || r < ng) {
          lo_w = *reinterpret_cast<const uint32_t*>(qbase + (size_t)r * QS + kk * 16 + 2 * t);
          hi_w = *reinterpret_cast<const uint32_t*>(qbase + (size_t)r * QS + kk * 16 + 8 + 2 * t);
        }
        qf[kk][h] = lo_w;
        qf[kk][2 + h] = hi_w;
      }
    }
  }

  int n = 0;
  for (int tile = first; tile < tile_end; tile += WARPS, ++n) {
    const int stage = n % DM_STAGES;
    const uint32_t parity = (n / DM_STAGES) & 1;
    if (!dm_bar_wait(&bars[warp][stage], parity)) { failed = true; break; }
    unsigned char* kt = my + (size_t)stage * 2 * TILE_BYTES;
    unsigned char* vt = kt + TILE_BYTES;
    const int k0 = lo_al + tile * DM_TK;
    // positions of the tile outside [lo, ctx): their value rows may hold anything; zero them
    if (k0 < lo || k0 + DM_TK > ctx) {
      const int row = lane & 15;
      const int kpos = k0 + row;
      if (kpos < lo || kpos >= ctx) {
        for (int c = (lane >> 4); c < D / 8; c += 2)
          *reinterpret_cast<uint4*>(vt + (c >> 3) * 2048 + row * 128 + ((c & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncwarp();
    }
    if constexpr (FUSED) {
      // the newest position is not in the cache yet (another CTA or this one writes it during
      // this very step): its rows of the tile come from shared memory
      const int r = ctx - 1 - k0;
      if (r >= 0 && r < DM_TK) {
        const int c = lane & 15;
        if (c < D / 8) {
          unsigned char* dst_t = (lane < 16) ? kt : vt;
          const bf16* srcp = new_kv + (lane < 16 ? 0 : D) + c * 8;
          *reinterpret_cast<uint4*>(dst_t + (c >> 3) * 2048 + r * 128 + (((c & 7) ^ (r & 7)) << 4)) =
              *reinterpret_cast<const uint4*>(srcp);
        }
        __syncwarp();
      }
    }
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
      const int chunk = kk * 2 + ((lane >> 3) & 1);
      dm_ldmatrix_x4(bfr, dm_swizzled(kt, key, chunk));
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
        const int chunk = dp * 2 + (lane >> 4);
        dm_ldmatrix_x4_trans(vfr, dm_swizzled(vt, key, chunk));
        dm_mma(o[2 * dp], pf, vfr[0], vfr[1]);
        dm_mma(o[2 * dp + 1], pf, vfr[2], vfr[3]);
      }
    }
    __syncwarp();                                  // every lane is done with this stage
    // order this warp's accesses to the stage (reads, and the zeroing above) before the copy
    // engine's next write into it
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    const int nxt = tile + DM_STAGES * WARPS;
    if (nxt < tile_end) load_tile(nxt, stage);
  }
  if (failed && lane == 0) atomicExch(error_flag, WAIT_FAILED_DECODE_TMA);

  // ---- row sums across the quad; then merge the warps through shared memory
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  __syncthreads();                                 // all warps are done with their tiles
  // [WARPS][16][D + 8], reusing the tile memory. A row is D sums, the maximum and the weight; rows
  // are D + 8 floats apart so that the 8-byte stores below (a half-warp: rows g = 0..3, column pairs
  // t = 0..3) fall into 16 different bank pairs (a stride of D + 2 put up to four lanes on one bank)
  float* red = reinterpret_cast<float*>(tiles);
  constexpr int WS = D + 8;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + 8 * h;
    if (r < ng) {
      float* w = red + ((size_t)warp * 16 + r) * WS;
#pragma unroll
      for (int i = 0; i < 2 * D16; ++i) {
        *reinterpret_cast<float2*>(w + i * 8 + 2 * t) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
      }
      if (t == 0) { w[D] = m[h]; w[D + 1] = l[h]; }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < ng * D; idx += (WARPS * 32)) {
    const int r = idx / D, d = idx - r * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, red[((size_t)w * 16 + r) * WS + D]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float* ws = red + ((size_t)w * 16 + r) * WS;
      const float c = (ws[D] == -INFINITY) ? 0.f : exp2f(ws[D] - mm);
      num += ws[d] * c;
      den += ws[D + 1] * c;
    }
    const int head = kvh * G + g0 + r;
    if (a.num_splits == 1) {
      ((bf16*)a.out)[((size_t)qrow * a.num_heads + head) * D + d] = __float2bfloat16_rn(num / den);
    } else if constexpr (CLUSTER) {
      const int S = a.num_splits, share = (ng * D + S - 1) / S;
      if (S * share <= RECV_CAP) {
        // straight into the shared memory of the CTA that merges this output (see below)
        const int owner = idx / share;
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(dm_smem(recv_num)), "r"(owner));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + 4u * (uint32_t)(split * share + idx - owner * share)), "f"(num) : "memory");
        if (d == 0) {
          for (int o2 = 0; o2 < S; ++o2) {
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(dm_smem(recv_ml)), "r"(o2));
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + 4u * (uint32_t)((split * 16 + r) * 2)), "f"(mm) : "memory");
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + 4u * (uint32_t)((split * 16 + r) * 2 + 1)), "f"(den) : "memory");
          }
        }
      } else {
        float* part = red + (size_t)WARPS * 16 * WS;          // [16][D + 8]: this range's sums, max and weight
        part[r * WS + d] = num;
        if (d == 0) { part[r * WS + D] = mm; part[r * WS + D + 1] = den; }
      }
    } else {
      const size_t pidx = ((size_t)si * a.num_heads + head) * a.num_splits + split;
      a.part_acc[pidx * D + d] = num;
      if (d == 0) { a.part_ml[pidx * 2] = mm; a.part_ml[pidx * 2 + 1] = den; }
    }
  }
  if (a.num_splits == 1) return;
  if constexpr (CLUSTER) {
    // ---- every CTA of the cluster merges its share of the outputs from all ranges' shared
    // memory, ranges in order (the sums of merge_splits, so both paths give the same bits)
    // Where the ranges' results fit into the receive buffers (small kv groups), every CTA has sent each
    // output to the CTA that merges it before this barrier, so that the merge reads its own shared
    // memory and a CTA may leave as soon as it has stored: measured with device clock stamps at batch 8,
    // pulling the results after the barrier cost 1,400 cycles of remote loads and a second cluster
    // barrier of 1,000 (nobody may leave while its shared memory can still be read) of a kernel of 20,000.
    const int S = a.num_splits;
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    const int total = ng * D;
    const int share = (total + S - 1) / S;
    const int end = min(total, (split + 1) * share);
    if (S * share <= RECV_CAP) {
      for (int idx = split * share + threadIdx.x; idx < end; idx += WARPS * 32) {
        const int r = idx / D, d = idx - r * D;
        float v[8], ms[8], ls[8];
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) {
          v[sp] = 0.f; ms[sp] = -INFINITY; ls[sp] = 0.f;
          if (sp < S) {
            v[sp] = recv_num[sp * share + idx - split * share];
            ms[sp] = recv_ml[(sp * 16 + r) * 2];
            ls[sp] = recv_ml[(sp * 16 + r) * 2 + 1];
          }
        }
        float mm = -INFINITY;
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) mm = fmaxf(mm, ms[sp]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) {
          if (sp < S) {
            const float c = (ms[sp] == -INFINITY) ? 0.f : exp2f(ms[sp] - mm);
            num += v[sp] * c;
            den += ls[sp] * c;
          }
        }
        ((bf16*)a.out)[((size_t)qrow * a.num_heads + kvh * G + g0 + r) * D + d] = __float2bfloat16_rn(num / den);
      }
      return;
    }
    const uint32_t part_addr = dm_smem(red + (size_t)WARPS * 16 * WS);
    for (int idx = split * share + threadIdx.x; idx < end; idx += WARPS * 32) {
      const int r = idx / D, d = idx - r * D;
      float v[8], ms[8], ls[8];
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) {
        v[sp] = 0.f; ms[sp] = -INFINITY; ls[sp] = 0.f;
        if (sp < S) {
          uint32_t remote;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(part_addr), "r"(sp));
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[sp]) : "r"(remote + 4u * (uint32_t)(r * WS + d)));
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(ms[sp]) : "r"(remote + 4u * (uint32_t)(r * WS + D)));
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(ls[sp]) : "r"(remote + 4u * (uint32_t)(r * WS + D + 1)));
        }
      }
      float mm = -INFINITY;
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) mm = fmaxf(mm, ms[sp]);
      float num = 0.f, den = 0.f;
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) {
        if (sp < S) {
          const float c = (ms[sp] == -INFINITY) ? 0.f : exp2f(ms[sp] - mm);
          num += v[sp] * c;
          den += ls[sp] * c;
        }
      }
      ((bf16*)a.out)[((size_t)qrow * a.num_heads + kvh * G + g0 + r) * D + d] = __float2bfloat16_rn(num / den);
    }
    // nobody leaves while another CTA may still read its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    return;
  }
  // ---- the CTA that arrives last for this (request, heads) merges the ranges
  unsigned int* counter = &g_dt_arrivals[((size_t)si * gridDim.y + blockIdx.y) % DM_MAX_COUNTERS];
  if (!cta_arrives_last(counter, (unsigned int)a.num_splits, &is_last)) return;
  merge_splits<bf16>(a, si, qrow, kvh * G + g0, ng, red);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*DtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static DtEncodeFn dt_encode_fn() {
  static DtEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (DtEncodeFn)p;
  }
  return fn;
}

// The descriptor of one cache tensor ([rows, head_dim] bf16, boxes of box_rows x 64, 128-byte
// swizzle). Descriptors are kept per (address, rows, head_dim, box_rows): a cache tensor is
// allocated once and used for every step.
static const CUtensorMap* cache_map(const void* base, long long rows, int head_dim, int box_rows) {
  static std::mutex mu;
  static std::map<std::tuple<const void*, long long, int, int>, CUtensorMap> maps;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_tuple(base, rows, head_dim, box_rows);
  auto it = maps.find(key);
  if (it != maps.end()) return &it->second;
  DtEncodeFn fn = dt_encode_fn();
  if (fn == nullptr) return nullptr;
  CUtensorMap m;
  cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return nullptr;
  return &maps.emplace(key, m).first->second;
}

static int g_decode_cluster_merge = 1;

template <int D64, int BR, bool FUSED, int WARPS, bool CLUSTER>
static int launch_dt_w(const AttnArgs& a, long long cache_rows, int* error_flag, cudaStream_t stream, const FusedQkv& f) {
  constexpr int D = D64 * 64;
  const CUtensorMap* mk = cache_map(a.k_cache, cache_rows, D, BR);
  const CUtensorMap* mv = cache_map(a.v_cache, cache_rows, D, BR);
  if (mk == nullptr || mv == nullptr) return TS_ERR_UNSUPPORTED;
  const size_t tiles = (size_t)WARPS * DM_STAGES * 2 * DM_TK * D * 2 + 1024;
  const size_t red = sizeof(float) * (size_t)(WARPS + 1) * 16 * (D + 8) + 1024;     // the warps' results and the CTA's
  const size_t smem = tiles > red ? tiles : red;
  auto kern = decode_attn_tma_kernel<D64, BR, FUSED, WARPS, CLUSTER>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int G = a.num_heads / a.num_kv_heads;
  const int passes = (G + 15) / 16;
  if (a.num_splits > 1 && (long long)a.num_seqs * a.num_kv_heads * passes > DM_MAX_COUNTERS) return TS_ERR_UNSUPPORTED;
  dim3 grid(a.num_seqs, a.num_kv_heads * passes, a.num_splits);
  if (CLUSTER)
    return launch_cluster(kern, grid, WARPS * 32, smem, stream, dim3(1, 1, a.num_splits), *mk, *mv, a, f, passes,
                          error_flag);
  return launch(kern, grid, WARPS * 32, smem, stream, *mk, *mv, a, f, passes, error_flag);
}

// Four warps per CTA run three to an SM (registers, shared memory); an unsplit grid of more than
// 3 x 148 and at most 4 x 148 CTAs would need a second, nearly empty round of them, so it gets
// CTAs of three warps, four to an SM (batch 64 of the 16 / 8 head layout: 512 CTAs).
template <int D64, int BR, bool FUSED = false>
static int launch_dt(const AttnArgs& a, long long cache_rows, int* error_flag, cudaStream_t stream,
                     const FusedQkv& f = FusedQkv()) {
  const int G = a.num_heads / a.num_kv_heads;
  const long long ctas = (long long)a.num_seqs * a.num_kv_heads * ((G + 15) / 16) * a.num_splits;
  if (D64 == 2 && a.num_splits == 1 && ctas > 3 * 148 && ctas <= 4 * 148)
    return launch_dt_w<D64, BR, FUSED, 3, false>(a, cache_rows, error_flag, stream, f);
  // 2 to 8 key ranges (the portable cluster size) merge inside a cluster
  if (g_decode_cluster_merge && a.num_splits >= 2 && a.num_splits <= 8)
    return launch_dt_w<D64, BR, FUSED, 4, true>(a, cache_rows, error_flag, stream, f);
  return launch_dt_w<D64, BR, FUSED, 4, false>(a, cache_rows, error_flag, stream, f);
}

}  // namespace ts

using namespace ts;

// Whether 2 to 8 key ranges are merged inside a thread-block cluster (on by default) or through
// global memory like larger numbers of ranges; both give the same bits.
extern "C" void ts_set_decode_cluster_merge(int on) { g_decode_cluster_merge = on; }

// bf16 decode attention with TMA tile loads. head_dim 64 or 128; page_size 8 or a multiple of 16;
// num_pages_total = pages of the cache tensors (the pad page included). Other arguments as
// ts_decode_attention_mma. Returns TS_ERR_UNSUPPORTED for sizes it does not take.
extern "C" int ts_decode_attention_tma(
    const void* q, void* out, const void* k_cache, const void* v_cache, long long num_pages_total,
    const int* block_tables, int table_width, const int* cu_q, const int* ctx_lens, const int* decode_seqs,
    int num_decode, int num_heads, int num_kv_heads, int head_dim, int page_size, float scale, int window,
    int num_splits, float* part_acc, float* part_ml, int* error_flag, cudaStream_t stream) {
  if (num_decode <= 0) return 0;
  if ((head_dim != 64 && head_dim != 128) || error_flag == nullptr) return TS_ERR_UNSUPPORTED;
  if (!(page_size == 8 || (page_size > 0 && page_size % 16 == 0))) return TS_ERR_UNSUPPORTED;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || window < 0 || num_splits < 1 || num_splits > ATTN_MAX_SPLITS || num_pages_total <= 0)
    return TS_ERR_BAD_ARGUMENT;
  if (num_splits > 1 && (part_acc == nullptr || part_ml == nullptr)) return TS_ERR_BAD_ARGUMENT;
  if ((((uintptr_t)k_cache) | ((uintptr_t)v_cache)) & 15) return TS_ERR_UNSUPPORTED;
  const long long rows = num_pages_total * num_kv_heads * page_size;
  if (rows >= (1ll << 31)) return TS_ERR_UNSUPPORTED;
  AttnArgs a;
  a.q = q; a.out = out; a.k_cache = k_cache; a.v_cache = v_cache;
  a.block_tables = block_tables; a.table_width = table_width; a.cu_q = cu_q; a.ctx_lens = ctx_lens;
  a.seq_ids = decode_seqs; a.num_seqs = num_decode;
  a.num_heads = num_heads; a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.page_size = page_size;
  a.page_shift = page_shift_of(page_size);
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  a.num_splits = num_splits; a.part_acc = part_acc; a.part_ml = part_ml;
  if (head_dim == 64) {
    return page_size == 8 ? launch_dt<1, 8>(a, rows, error_flag, stream) : launch_dt<1, 16>(a, rows, error_flag, stream);
  }
  return page_size == 8 ? launch_dt<2, 8>(a, rows, error_flag, stream) : launch_dt<2, 16>(a, rows, error_flag, stream);
}

// The same attention for a step of decode tokens only, fed with the raw output of the qkv product:
// the kernel normalises (per-head RMSNorm; a null weight skips it) and rotates (rotate-half over
// the whole head; null tables skip it) the queries and the new key itself, stores the new key and
// value at `slots`, and attends over the cache with them. qkv is [tokens, (num_heads +
// 2 num_kv_heads) * head_dim]; cos_t/sin_t are [tokens, head_dim / 2]; a request's token is row
// cu_q[request]. Replaces ts_qk_norm_rope_write followed by ts_decode_attention_tma.
extern "C" int ts_decode_attention_tma_fused(
    const void* qkv, const void* q_weight, const void* k_weight, float eps, const float* cos_t, const float* sin_t,
    const int* slots, void* out, void* k_cache, void* v_cache, long long num_pages_total, const int* block_tables,
    int table_width, const int* cu_q, const int* ctx_lens, const int* decode_seqs, int num_decode, int num_heads,
    int num_kv_heads, int head_dim, int page_size, float scale, int window, int num_splits, float* part_acc,
    float* part_ml, int* error_flag, cudaStream_t stream) {
  if (num_decode <= 0) return 0;
  if ((head_dim != 64 && head_dim != 128) || error_flag == nullptr) return TS_ERR_UNSUPPORTED;
  if (!(page_size == 8 || (page_size > 0 && page_size % 16 == 0))) return TS_ERR_UNSUPPORTED;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || window < 0 || num_splits < 1 || num_splits > ATTN_MAX_SPLITS || num_pages_total <= 0)
    return TS_ERR_BAD_ARGUMENT;
  if (num_splits > 1 && (part_acc == nullptr || part_ml == nullptr)) return TS_ERR_BAD_ARGUMENT;
  if ((cos_t == nullptr) != (sin_t == nullptr) || slots == nullptr || qkv == nullptr) return TS_ERR_BAD_ARGUMENT;
  if ((((uintptr_t)k_cache) | ((uintptr_t)v_cache) | ((uintptr_t)qkv)) & 15) return TS_ERR_UNSUPPORTED;
  const long long rows = num_pages_total * num_kv_heads * page_size;
  if (rows >= (1ll << 31)) return TS_ERR_UNSUPPORTED;
  AttnArgs a;
  a.q = nullptr; a.out = out; a.k_cache = k_cache; a.v_cache = v_cache;
  a.block_tables = block_tables; a.table_width = table_width; a.cu_q = cu_q; a.ctx_lens = ctx_lens;
  a.seq_ids = decode_seqs; a.num_seqs = num_decode;
  a.num_heads = num_heads; a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.page_size = page_size;
  a.page_shift = page_shift_of(page_size);
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  a.num_splits = num_splits; a.part_acc = part_acc; a.part_ml = part_ml;
  FusedQkv f;
  f.qkv = (const bf16*)qkv; f.q_weight = (const bf16*)q_weight; f.k_weight = (const bf16*)k_weight; f.eps = eps;
  f.cos_t = cos_t; f.sin_t = sin_t; f.slots = slots; f.k_cache = (bf16*)k_cache; f.v_cache = (bf16*)v_cache;
  if (head_dim == 64) {
    return page_size == 8 ? launch_dt<1, 8, true>(a, rows, error_flag, stream, f)
                          : launch_dt<1, 16, true>(a, rows, error_flag, stream, f);
  }
  return page_size == 8 ? launch_dt<2, 8, true>(a, rows, error_flag, stream, f)
                        : launch_dt<2, 16, true>(a, rows, error_flag, stream, f);
}

// How many CTAs of this kernel fit the machine at once (for the split choice).
extern "C" int ts_decode_attention_tma_slots(int head_dim) {
  const size_t smem = (size_t)DM_WARPS * DM_STAGES * 2 * DM_TK * head_dim * 2 + 2048;
  int per_sm = (int)((227 * 1024) / smem);
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 3) per_sm = 3;       // registers: 160 per thread
  return 148 * per_sm;
}
