// Varlen causal prefill attention over the paged cache on the tensor cores (bf16) with TMA tile
// loads: head sizes 64 and 128, page sizes 8 or a multiple of 16. Math and tiling as in
// attention_mma.cu (upstream src/tinyserve/attention.py:89-111, src/tinyserve/triton_prefill.py:50-125);
// this variant is built for occupancy and balance:
//  * keys and values come in tiles of 32 positions fetched by one thread with cp.async.bulk.tensor
//    (boxes of 16 or 8 cache rows by 64 columns, 128-byte swizzled, mbarrier completion), so the
//    other threads issue no copy instructions and shared memory needs no padding;
//  * query fragments are re-read from shared memory for every tile instead of living in
//    registers, which keeps a CTA at 128 registers per thread and 48 KiB: four CTAs per SM;
//  * a CTA takes a pair of 64-row query tiles of one request, the i-th and the i-th from the end,
//    so under the causal mask every CTA of a request does the same amount of work.
// A row of a query tile is a (token, query head of the kv group) pair, as in attention_mma.cu.
// Every mbarrier wait is bounded; a wait that runs out sets *error_flag and the CTA leaves.
#define TS_PDL_CLASS PDL_ATTENTION
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "attention.cuh"
#include "bounded_wait.cuh"

namespace ts {

constexpr int PT_BM = 64, PT_BN = 32, PT_THREADS = 128, PT_STAGES = 2;

__device__ __forceinline__ uint32_t pt_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pt_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(pt_smem(p)));
}
__device__ __forceinline__ void pt_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(pt_smem(p)));
}
__device__ __forceinline__ void pt_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pt_pack(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void pt_bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pt_smem(bar)), "r"(count));
}
__device__ __forceinline__ void pt_bar_arrive_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pt_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool pt_bar_wait(uint64_t* bar, uint32_t parity) {
  return bounded_mbar_wait(pt_smem(bar), parity);
}
__device__ __forceinline__ void pt_tensor_copy(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(pt_smem(dst)), "l"(map), "r"(pt_smem(bar)), "r"(x), "r"(y) : "memory");
}
// 16-byte chunk `chunk` (of head_dim / 8) of row `row` of a tile of ROWS rows stored as
// head_dim / 64 sub-tiles of ROWS x 128 bytes with the 128-byte swizzle.
template <int ROWS>
__device__ __forceinline__ unsigned char* pt_swizzled(unsigned char* tile, int row, int chunk) {
  return tile + (chunk >> 3) * (ROWS * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

// D64 = head_dim / 64; BR = rows of a tensor box (16, or 8 for pages of 8).
// `ge` = query heads per row group (the GQA group if it divides 64, else 1);
// blockIdx = (pair of query tiles, request in the list, kv head or query head).
template <int D64, int BR>
__global__ void __launch_bounds__(PT_THREADS, 4) prefill_attn_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                         const __grid_constant__ CUtensorMap map_v,
                                                                         AttnArgs a, int ge, int pair, int* error_flag) {
  constexpr int D = D64 * 64, D16 = D / 16, CH = D / 8;
  constexpr int Q_BYTES = PT_BM * D * 2, KV_BYTES = PT_BN * D * 2;
  extern __shared__ __align__(16) unsigned char pt_raw[];
  __shared__ __align__(8) uint64_t full_bar[PT_STAGES];
  pdl_trigger();
  unsigned char* base = (unsigned char*)(((uintptr_t)pt_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* Qs = base;                               // [D64][64 rows][128 B], swizzled
  unsigned char* KVs = base + Q_BYTES;                    // [stage][K|V][D64][32 rows][128 B]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  if (tid == 0) {
    for (int s = 0; s < PT_STAGES; ++s) pt_bar_init(&full_bar[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();

  const int group = a.num_heads / a.num_kv_heads;
  const int seq = a.seq_ids[blockIdx.y];
  const int head0 = (ge == group) ? blockIdx.z * group : blockIdx.z;
  const int kvh = head0 / group;
  const int row0 = a.cu_q[seq];
  const int n = a.cu_q[seq + 1] - row0;
  const int tpt = PT_BM / ge;                            // tokens per query tile
  const int ntiles_q = (n + tpt - 1) / tpt;
  if ((int)blockIdx.x * (pair ? 2 : 1) >= ntiles_q) return;
  const int ctx = a.ctx_lens[seq];
  const int first_pos = ctx - n;
  const int* table = a.block_tables + (size_t)seq * a.table_width;
  const bf16* q = (const bf16*)a.q;
  bf16* out = (bf16*)a.out;
  int it = 0;                                            // key tiles fetched so far (stage and phase)
  bool failed = false;

  for (int half = 0; half < (pair ? 2 : 1) && !failed; ++half) {
    // paired: the i-th tile and the i-th from the end; unpaired: one tile, the last ones (most
    // keys) launched first
    const int qt = pair ? ((half == 0) ? (int)blockIdx.x : ntiles_q - 1 - (int)blockIdx.x)
                        : ntiles_q - 1 - (int)blockIdx.x;
    if (half == 1 && qt <= (int)blockIdx.x) break;       // the middle tile of an odd count was done
    const int q0 = qt * tpt;
    const int ntok = min(tpt, n - q0);
    const int nrows = ntok * ge;
    const int qpos_first = first_pos + q0;
    const int qpos_last = first_pos + q0 + ntok - 1;
    const int k_lo = (a.window > 0) ? max(0, qpos_first - a.window + 1) : 0;
    const int k_begin = (k_lo / PT_BN) * PT_BN;
    const int num_tiles = (qpos_last - k_begin) / PT_BN + 1;

    auto load_tile = [&](int tile, int slot) {            // thread 0 only
      if (wait_test_unarmed()) return;
      const int k0 = k_begin + tile * PT_BN;
      unsigned char* kd = KVs + (size_t)slot * 2 * KV_BYTES;
      unsigned char* vd = kd + KV_BYTES;
      uint64_t* bar = &full_bar[slot];
      pt_bar_arrive_tx(bar, 2u * KV_BYTES);
#pragma unroll
      for (int part = 0; part < PT_BN / BR; ++part) {
        int kpos = k0 + part * BR;
        if (kpos >= ctx) kpos = k0;                      // wholly past the end: any valid rows, masked
        int page, off;
        if (a.page_shift >= 0) { page = table[kpos >> a.page_shift]; off = kpos & (a.page_size - 1); }
        else { const int idx = kpos / a.page_size; page = table[idx]; off = kpos - idx * a.page_size; }
        const int y = (page * a.num_kv_heads + kvh) * a.page_size + off;
#pragma unroll
        for (int h = 0; h < D64; ++h) {
          pt_tensor_copy(kd + h * (PT_BN * 128) + part * BR * 128, &map_k, h * 64, y, bar);
          pt_tensor_copy(vd + h * (PT_BN * 128) + part * BR * 128, &map_v, h * 64, y, bar);
        }
      }
    };

    __syncthreads();                                      // the previous half is done with Qs and the stages
    if (tid == 0) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      for (int s = 0; s < PT_STAGES && s < num_tiles; ++s) load_tile(s, (it + s) % PT_STAGES);
    }
    // ---- stage Q (row r = token q0 + r / ge, head head0 + r % ge), swizzled like the K/V tiles
    for (int idx = tid; idx < PT_BM * CH; idx += PT_THREADS) {
      const int r = idx / CH, c = idx - r * CH;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < nrows) {
        const int tok = q0 + r / ge, head = head0 + r % ge;
        v = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + tok) * a.num_heads + head) * D + c * 8);
      }
      *reinterpret_cast<uint4*>(pt_swizzled<PT_BM>(Qs, r, c)) = v;
    }
    __syncthreads();

    int qpos[2];
    bool rvalid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = warp * 16 + g + 8 * h;
      rvalid[h] = r < nrows;
      qpos[h] = first_pos + q0 + r / ge;
    }
    const int warp_last_row = min(warp * 16 + 15, nrows - 1);
    const int warp_qpos_max = first_pos + q0 + max(warp_last_row, 0) / ge;
    const int warp_qpos_min = first_pos + q0 + (warp * 16) / ge;
    const bool warp_active = warp * 16 < nrows;

    float o[2 * D16][4];
#pragma unroll
    for (int i = 0; i < 2 * D16; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int tile = 0; tile < num_tiles; ++tile, ++it) {
      const int slot = it % PT_STAGES;
      if (!pt_bar_wait(&full_bar[slot], (it / PT_STAGES) & 1)) { failed = true; break; }
      unsigned char* kt = KVs + (size_t)slot * 2 * KV_BYTES;
      unsigned char* vt = kt + KV_BYTES;
      const int k0 = k_begin + tile * PT_BN;
      // value rows of positions the request does not own (past its end, or before the window on
      // pages already given back) may hold anything: zero them
      if (k0 < k_lo || k0 + PT_BN > ctx) {
        for (int idx = tid; idx < PT_BN * CH; idx += PT_THREADS) {
          const int r = idx / CH, c = idx - r * CH;
          const int kpos = k0 + r;
          if (kpos < k_lo || kpos >= ctx)
            *reinterpret_cast<uint4*>(pt_swizzled<PT_BN>(vt, r, c)) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncthreads();
      }
      if (warp_active && k0 <= warp_qpos_max) {
        // ---- S = Q K^T : 4 key tiles of 8
        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D16; ++kk) {
          uint32_t qf[4];
          pt_ldmatrix_x4(qf, pt_swizzled<PT_BM>(Qs, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, kk * 2 + (lane >> 4)));
#pragma unroll
          for (int np = 0; np < 2; ++np) {
            uint32_t bfr[4];
            pt_ldmatrix_x4(bfr, pt_swizzled<PT_BN>(kt, np * 16 + (lane & 7) + (lane >> 4) * 8, kk * 2 + ((lane >> 3) & 1)));
            pt_mma(s[2 * np], qf, bfr[0], bfr[1]);
            pt_mma(s[2 * np + 1], qf, bfr[2], bfr[3]);
          }
        }
        // ---- scale, mask, online softmax (a tile that every row of the warp sees whole needs no mask)
        float mx[2] = {-INFINITY, -INFINITY};
        const bool whole = (k0 + PT_BN - 1 <= warp_qpos_min) && (a.window == 0 || k0 > warp_qpos_max - a.window);
        if (whole) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float v = s[i][e] * a.scale_log2;
              s[i][e] = v;
              mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int h = e >> 1;
              const int kpos = k0 + i * 8 + 2 * t + (e & 1);
              bool ok = rvalid[h] && kpos <= qpos[h];
              if (a.window > 0) ok = ok && (kpos > qpos[h] - a.window);
              const float v = ok ? s[i][e] * a.scale_log2 : -INFINITY;
              s[i][e] = v;
              mx[h] = fmaxf(mx[h], v);
            }
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
        for (int i = 0; i < 4; ++i)
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
        // ---- O += P V : 2 steps of 16 keys
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          uint32_t pf[4];
          pf[0] = pt_pack(s[2 * ks][0], s[2 * ks][1]);
          pf[1] = pt_pack(s[2 * ks][2], s[2 * ks][3]);
          pf[2] = pt_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]);
          pf[3] = pt_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
          for (int dp = 0; dp < D16; ++dp) {
            uint32_t vfr[4];
            pt_ldmatrix_x4_trans(vfr, pt_swizzled<PT_BN>(vt, ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + (lane >> 4)));
            pt_mma(o[2 * dp], pf, vfr[0], vfr[1]);
            pt_mma(o[2 * dp + 1], pf, vfr[2], vfr[3]);
          }
        }
      }
      __syncthreads();                                    // the stage is free
      if (tid == 0 && tile + PT_STAGES < num_tiles) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        load_tile(tile + PT_STAGES, slot);
      }
    }
    if (failed) break;

    // ---- normalise and write
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float ls = l[h];
      ls += __shfl_xor_sync(0xffffffffu, ls, 1);
      ls += __shfl_xor_sync(0xffffffffu, ls, 2);
      const int r = warp * 16 + g + 8 * h;
      if (r < nrows) {
        const float inv = 1.f / ls;
        const int tok = q0 + r / ge, head = head0 + r % ge;
        bf16* dst = out + ((size_t)(row0 + tok) * a.num_heads + head) * D;
#pragma unroll
        for (int i = 0; i < 2 * D16; ++i)
          *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) = pt_pack(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
      }
    }
  }
  if (failed && lane == 0) atomicExch(error_flag, WAIT_FAILED_PREFILL_TMA);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*PtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static const CUtensorMap* pt_cache_map(const void* base, long long rows, int head_dim, int box_rows) {
  static std::mutex mu;
  static std::map<std::tuple<const void*, long long, int, int>, CUtensorMap> maps;
  static PtEncodeFn fn = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_tuple(base, rows, head_dim, box_rows);
  auto it = maps.find(key);
  if (it != maps.end()) return &it->second;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = (PtEncodeFn)p;
  }
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

template <int D64, int BR>
static int launch_pt(const AttnArgs& a, long long cache_rows, int max_query_len, int* error_flag, cudaStream_t stream) {
  constexpr int D = D64 * 64;
  const CUtensorMap* mk = pt_cache_map(a.k_cache, cache_rows, D, BR);
  const CUtensorMap* mv = pt_cache_map(a.v_cache, cache_rows, D, BR);
  if (mk == nullptr || mv == nullptr) return TS_ERR_UNSUPPORTED;
  const size_t smem = (size_t)PT_BM * D * 2 + (size_t)PT_STAGES * 2 * PT_BN * D * 2 + 1024;
  auto kern = prefill_attn_tma_kernel<D64, BR>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int group = a.num_heads / a.num_kv_heads;
  const int ge = (group <= PT_BM && PT_BM % group == 0) ? group : 1;
  const int tpt = PT_BM / ge;
  const int ntiles_q = (max_query_len + tpt - 1) / tpt;
  const int grid_z = ge == group ? a.num_kv_heads : a.num_heads;
  // Pair the tiles (equal work per CTA) only if the pairs alone fill the machine twice over;
  // otherwise more, unequal CTAs keep more SMs busy.
  const int pair = ((long long)((ntiles_q + 1) / 2) * a.num_seqs * grid_z >= 2ll * 148 * 4) ? 1 : 0;
  dim3 grid(pair ? (ntiles_q + 1) / 2 : ntiles_q, a.num_seqs, grid_z);
  return launch(kern, grid, PT_THREADS, smem, stream, *mk, *mv, a, ge, pair, error_flag);
}

}  // namespace ts

using namespace ts;

// bf16 prefill attention with TMA tile loads for the requests listed in prefill_seqs. head_dim 64
// or 128; page_size 8 or a multiple of 16; num_pages_total = pages of the cache tensors (the pad
// page included). Returns TS_ERR_UNSUPPORTED for sizes it does not take.
extern "C" int ts_prefill_attention_tma(
    const void* q, void* out, const void* k_cache, const void* v_cache, long long num_pages_total,
    const int* block_tables, int table_width, const int* cu_q, const int* ctx_lens, const int* prefill_seqs,
    int num_prefill, int max_query_len, int num_heads, int num_kv_heads, int head_dim, int page_size, float scale,
    int window, int* error_flag, cudaStream_t stream) {
  if (num_prefill <= 0) return 0;
  if ((head_dim != 64 && head_dim != 128) || error_flag == nullptr) return TS_ERR_UNSUPPORTED;
  if (!(page_size == 8 || (page_size > 0 && page_size % 16 == 0))) return TS_ERR_UNSUPPORTED;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || window < 0 || num_pages_total <= 0) return TS_ERR_BAD_ARGUMENT;
  if ((((uintptr_t)k_cache) | ((uintptr_t)v_cache) | ((uintptr_t)q)) & 15) return TS_ERR_UNSUPPORTED;
  const long long rows = num_pages_total * num_kv_heads * page_size;
  if (rows >= (1ll << 31)) return TS_ERR_UNSUPPORTED;
  AttnArgs a;
  a.q = q; a.out = out; a.k_cache = k_cache; a.v_cache = v_cache;
  a.block_tables = block_tables; a.table_width = table_width; a.cu_q = cu_q; a.ctx_lens = ctx_lens;
  a.seq_ids = prefill_seqs; a.num_seqs = num_prefill;
  a.num_heads = num_heads; a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.page_size = page_size;
  a.page_shift = page_shift_of(page_size);
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  a.num_splits = 1; a.part_acc = nullptr; a.part_ml = nullptr;
  if (head_dim == 64)
    return page_size == 8 ? launch_pt<1, 8>(a, rows, max_query_len, error_flag, stream)
                          : launch_pt<1, 16>(a, rows, max_query_len, error_flag, stream);
  return page_size == 8 ? launch_pt<2, 8>(a, rows, max_query_len, error_flag, stream)
                        : launch_pt<2, 16>(a, rows, max_query_len, error_flag, stream);
}
