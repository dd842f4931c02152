// Varlen causal prefill attention over the paged cache on the tensor cores (bf16), for head
// sizes of 16..128 in steps of 16. Math as in attention_simt.cu (upstream
// src/tinyserve/attention.py:89-111; the tiling over the paged cache and the rounding of the
// probabilities to the value type before the second product follow upstream
// src/tinyserve/triton_prefill.py:50-125).
//
// One CTA = 64 query rows x one kv head. A row is a (token, query head of the group) pair, so
// the heads that share a kv head share every key and value tile that is staged. Keys and values
// come in tiles of 64 positions, fetched page by page with 16-byte cp.async into padded shared
// memory (row stride head_dim + 8 elements: ldmatrix reads without bank conflicts for every head
// size) and double-buffered. S = Q K^T and O += P V are mma.sync m16n8k16 with 32-bit
// accumulators; the softmax is online, in 32-bit, base 2.
#define TS_PDL_CLASS PDL_ATTENTION
#include <cuda_pipeline_primitives.h>

#include "attention.cuh"

namespace ts {

constexpr int MA_BM = 64, MA_BN = 64, MA_THREADS = 128;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_ptr) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// D16 = head_dim / 16. `ge` = query heads per row group (the GQA group if it divides 64, else 1);
// blockIdx.z = kv head when ge == group, else query head.
template <int D16>
__global__ void __launch_bounds__(MA_THREADS) prefill_attn_mma_kernel(AttnArgs a, int ge) {
  constexpr int D = D16 * 16, DS = D + 8, CH = D / 8;   // CH = 16-byte chunks per row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);          // [64][DS]
  bf16* Ks = Qs + MA_BM * DS;                            // [2][64][DS]
  bf16* Vs = Ks + 2 * MA_BN * DS;                        // [2][64][DS]

  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int group = a.num_heads / a.num_kv_heads;
  const int seq = a.seq_ids[blockIdx.y];
  const int head0 = (ge == group) ? blockIdx.z * group : blockIdx.z;
  const int kvh = head0 / group;
  const int row0 = a.cu_q[seq];
  const int n = a.cu_q[seq + 1] - row0;
  const int tpt = MA_BM / ge;                            // tokens per tile
  // the tiles with the most keys (the last queries) are launched first, so the partly filled
  // last round of CTAs is made of the cheapest ones
  const int q0 = (int)(gridDim.x - 1 - blockIdx.x) * tpt;
  if (q0 >= n) return;
  const int ctx = a.ctx_lens[seq];
  const int first_pos = ctx - n;
  const int ntok = min(tpt, n - q0);
  const int nrows = ntok * ge;
  const int* table = a.block_tables + (size_t)seq * a.table_width;
  const bf16* q = (const bf16*)a.q;
  const bf16* kc = (const bf16*)a.k_cache;
  const bf16* vc = (const bf16*)a.v_cache;

  const int qpos_first = first_pos + q0;
  const int qpos_last = first_pos + q0 + ntok - 1;
  const int k_lo = (a.window > 0) ? max(0, qpos_first - a.window + 1) : 0;
  const int k_begin = (k_lo / MA_BN) * MA_BN;
  const int num_tiles = (qpos_last - k_begin) / MA_BN + 1;

  // ---- stage Q (row r = token q0 + r / ge, head head0 + r % ge)
  for (int idx = tid; idx < MA_BM * CH; idx += MA_THREADS) {
    const int r = idx / CH, c = idx - r * CH;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < nrows) {
      const int tok = q0 + r / ge, head = head0 + r % ge;
      v = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + tok) * a.num_heads + head) * D + c * 8);
    }
    *reinterpret_cast<uint4*>(Qs + r * DS + c * 8) = v;
  }

  auto load_tile = [&](int tile, int buf) {
    const int k0 = k_begin + tile * MA_BN;
    bf16* kd = Ks + buf * MA_BN * DS;
    bf16* vd = Vs + buf * MA_BN * DS;
    for (int idx = tid; idx < MA_BN * CH; idx += MA_THREADS) {
      const int kk = idx / CH, c = idx - kk * CH;
      const int kpos = k0 + kk;
      if (kpos >= k_lo && kpos <= qpos_last) {
        const size_t off = kv_offset_of(table, kpos, kvh, a) + (size_t)c * 8;
        __pipeline_memcpy_async(kd + kk * DS + c * 8, kc + off, 16);
        __pipeline_memcpy_async(vd + kk * DS + c * 8, vc + off, 16);
      } else {
        *reinterpret_cast<uint4*>(kd + kk * DS + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(vd + kk * DS + c * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    __pipeline_commit();
  };

  load_tile(0, 0);
  __syncthreads();   // Qs is complete

  // ---- Q fragments of this warp's 16 rows
  uint32_t qf[D16][4];
#pragma unroll
  for (int kk = 0; kk < D16; ++kk) {
    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int c = kk * 16 + (lane >> 4) * 8;
    ldmatrix_x4(qf[kk], Qs + r * DS + c);
  }

  // rows of this thread: warp * 16 + g and + 8
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
  const bool warp_active = warp * 16 < nrows;
  const int warp_qpos_min = first_pos + q0 + (warp * 16) / ge;

  float o[2 * D16][4];
#pragma unroll
  for (int i = 0; i < 2 * D16; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int tile = 0; tile < num_tiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < num_tiles) load_tile(tile + 1, buf ^ 1);
    if (tile + 1 < num_tiles) __pipeline_wait_prior(1); else __pipeline_wait_prior(0);
    __syncthreads();
    const int k0 = k_begin + tile * MA_BN;
    if (warp_active && k0 <= warp_qpos_max) {
      const bf16* kt = Ks + buf * MA_BN * DS;
      const bf16* vt = Vs + buf * MA_BN * DS;
      // ---- S = Q K^T : 8 key tiles of 8
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
#pragma unroll
      for (int kk = 0; kk < D16; ++kk) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {       // pairs of key tiles
          uint32_t bfr[4];
          const int key = np * 16 + (lane & 7) + (lane >> 4) * 8;
          const int c = kk * 16 + ((lane >> 3) & 1) * 8;
          ldmatrix_x4(bfr, kt + key * DS + c);
          mma_16816(s[2 * np], qf[kk], bfr[0], bfr[1]);
          mma_16816(s[2 * np + 1], qf[kk], bfr[2], bfr[3]);
        }
      }
      // ---- scale, mask, online softmax. A tile that every row of the warp sees whole needs no
      //      mask (rows beyond the tile's last have zero queries and finite scores).
      float mx[2] = {-INFINITY, -INFINITY};
      const bool whole = (k0 + MA_BN - 1 <= warp_qpos_min) && (a.window == 0 || k0 > warp_qpos_max - a.window);
      if (whole) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float v = s[i][e] * a.scale_log2;
            s[i][e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
          }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
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
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          const float p = (s[i][e] == -INFINITY) ? 0.f : exp2f(s[i][e] - m[h]);
          s[i][e] = p;
          l[h] += p;
        }
#pragma unroll
      for (int i = 0; i < 2 * D16; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0];
        o[i][2] *= corr[1]; o[i][3] *= corr[1];
      }
      // ---- O += P V : 4 steps of 16 keys, D / 8 column tiles
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t pf[4];
        pf[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
        pf[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
        pf[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
        pf[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
        for (int dp = 0; dp < D16; ++dp) {     // pairs of column tiles (16 dims)
          uint32_t vfr[4];
          const int key = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int c = dp * 16 + (lane >> 4) * 8;
          ldmatrix_x4_trans(vfr, vt + key * DS + c);
          mma_16816(o[2 * dp], pf, vfr[0], vfr[1]);
          mma_16816(o[2 * dp + 1], pf, vfr[2], vfr[3]);
        }
      }
    }
    __syncthreads();   // the buffer is free for the load after next
  }

  // ---- normalise and write
  bf16* out = (bf16*)a.out;
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
      for (int i = 0; i < 2 * D16; ++i) {
        const uint32_t v = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
        *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) = v;
      }
    }
  }
}

template <int D16>
static int launch_mma(const AttnArgs& a, int max_query_len, cudaStream_t stream) {
  constexpr int DS = D16 * 16 + 8;
  const size_t smem = sizeof(bf16) * (size_t)(MA_BM + 4 * MA_BN) * DS;
  auto kern = prefill_attn_mma_kernel<D16>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int group = a.num_heads / a.num_kv_heads;
  const int ge = (group <= MA_BM && MA_BM % group == 0) ? group : 1;
  const int tpt = MA_BM / ge;
  dim3 grid((max_query_len + tpt - 1) / tpt, a.num_seqs, ge == group ? a.num_kv_heads : a.num_heads);
  return launch(kern, grid, MA_THREADS, smem, stream, a, ge);
}

}  // namespace ts

using namespace ts;

// bf16 prefill attention for the requests listed in prefill_seqs. head_dim in {16, 32, ..., 128}.
extern "C" int ts_prefill_attention_mma(
    const void* q, void* out, const void* k_cache, const void* v_cache, const int* block_tables,
    int table_width, const int* cu_q, const int* ctx_lens, const int* prefill_seqs, int num_prefill,
    int max_query_len, int num_heads, int num_kv_heads, int head_dim, int page_size, float scale,
    int window, cudaStream_t stream) {
  if (num_prefill <= 0) return 0;
  if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 128) return TS_ERR_UNSUPPORTED;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || page_size <= 0 || window < 0) return TS_ERR_BAD_ARGUMENT;
  AttnArgs a;
  a.q = q; a.out = out; a.k_cache = k_cache; a.v_cache = v_cache;
  a.block_tables = block_tables; a.table_width = table_width; a.cu_q = cu_q; a.ctx_lens = ctx_lens;
  a.seq_ids = prefill_seqs; a.num_seqs = num_prefill;
  a.num_heads = num_heads; a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.page_size = page_size;
  a.page_shift = page_shift_of(page_size);
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  a.num_splits = 1; a.part_acc = nullptr; a.part_ml = nullptr;
  switch (head_dim / 16) {
    case 1: return launch_mma<1>(a, max_query_len, stream);
    case 2: return launch_mma<2>(a, max_query_len, stream);
    case 3: return launch_mma<3>(a, max_query_len, stream);
    case 4: return launch_mma<4>(a, max_query_len, stream);
    case 5: return launch_mma<5>(a, max_query_len, stream);
    case 6: return launch_mma<6>(a, max_query_len, stream);
    case 7: return launch_mma<7>(a, max_query_len, stream);
    case 8: return launch_mma<8>(a, max_query_len, stream);
  }
  return TS_ERR_UNSUPPORTED;
}
