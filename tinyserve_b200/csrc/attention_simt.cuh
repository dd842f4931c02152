// Paged attention on CUDA cores (kernel templates and their launch helpers), for float and bf16: the true 32-bit path of the engine and
// the fallback for head sizes the tensor-core kernels do not take.
//
// Math (upstream src/tinyserve/attention.py:89-111): s = scale * q.k over head_dim in 32-bit,
// causal mask (key position <= query position; optionally > query position - window),
// softmax in 32-bit (online, base 2), o = sum p v in 32-bit, cast once to the output type.
// Query head h reads kv head h / (num_heads / num_kv_heads).
//
//  * prefill kernel: one CTA per (tile of 32 queries of one request, query head); keys and
//    values are staged through shared memory in tiles of 32 (after upstream
//    src/tinyserve/triton_prefill.py:50-125, which tiles the same way over the paged cache).
//  * decode kernel: one CTA per (request, kv head, split of the keys); a group of lanes reads
//    one key with 16-byte loads, all query heads of the group share each key and value; the
//    CTA that finishes last merges the splits (the split-K scheme is upstream's,
//    src/tinyserve/triton_attention.py:243-327, which merges in a second kernel).
// Keys outside a request's own range are never loaded: their scores are -inf and their values
// zero, so whatever lies in pages of other requests cannot reach the result.
#pragma once
#include "attention.cuh"

namespace ts {

constexpr float NEG_INF = -INFINITY;

// =============================================================== prefill (tiled)
constexpr int PF_TQ = 32;       // queries per CTA
constexpr int PF_TK = 32;       // keys per tile
constexpr int PF_THREADS = 128;

template <typename T, int DJMAX>
__global__ void __launch_bounds__(PF_THREADS) prefill_attn_kernel(AttnArgs a) {
  extern __shared__ float smem[];
  const int D = a.head_dim;
  const int DS = D + 1;                         // padded row stride
  float* Qs = smem;                             // [TQ][DS]  pre-scaled queries
  float* Ks = Qs + PF_TQ * DS;                  // [TK][DS]
  float* Vs = Ks + PF_TK * DS;                  // [TK][D]
  float* Ss = Vs + PF_TK * D;                   // [TQ][TK + 1]
  float* row_m = Ss + PF_TQ * (PF_TK + 1);      // [TQ]
  float* row_l = row_m + PF_TQ;                 // [TQ]
  float* row_c = row_l + PF_TQ;                 // [TQ] correction factor of this tile

  pdl_trigger();
  pdl_wait();
  const int seq = a.seq_ids[blockIdx.y];
  const int head = blockIdx.z;
  const int kvh = head / (a.num_heads / a.num_kv_heads);
  const int row0 = a.cu_q[seq];
  const int n = a.cu_q[seq + 1] - row0;
  const int q0 = blockIdx.x * PF_TQ;
  if (q0 >= n) return;
  const int ctx = a.ctx_lens[seq];
  const int first_pos = ctx - n;                // position of the request's first new token
  const int nq = min(PF_TQ, n - q0);
  const int* table = a.block_tables + (size_t)seq * a.table_width;
  const T* q = (const T*)a.q;
  const T* kc = (const T*)a.k_cache;
  const T* vc = (const T*)a.v_cache;
  const int tid = threadIdx.x;

  for (int idx = tid; idx < PF_TQ * D; idx += PF_THREADS) {
    const int r = idx / D, d = idx - r * D;
    float v = 0.f;
    if (r < nq) v = to_float(q[((size_t)(row0 + q0 + r) * a.num_heads + head) * D + d]) * a.scale_log2;
    Qs[r * DS + d] = v;
  }
  if (tid < PF_TQ) { row_m[tid] = NEG_INF; row_l[tid] = 0.f; }

  const int ty = tid >> 4, tx = tid & 15;       // 8 row groups x 16 column groups
  float acc[4][DJMAX];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < DJMAX; ++j) acc[i][j] = 0.f;
  const int dj = D >> 4;

  const int qpos_first = first_pos + q0;
  const int qpos_last = first_pos + q0 + nq - 1;
  int k_lo = 0;
  if (a.window > 0) k_lo = max(0, qpos_first - a.window + 1);
  const int k_begin = (k_lo / PF_TK) * PF_TK;
  constexpr int VEC = Vec<T>::N;
  const int chunks = D / VEC;

  for (int k0 = k_begin; k0 <= qpos_last; k0 += PF_TK) {
    __syncthreads();   // previous tile fully consumed (and Qs/row state initialised)
    // ---- stage keys and values k0 .. k0+TK-1 (zeros outside the request's visible range)
    for (int idx = tid; idx < PF_TK * chunks; idx += PF_THREADS) {
      const int kk = idx / chunks, c = idx - kk * chunks;
      const int kpos = k0 + kk;
      float kf[VEC], vf[VEC];
      if (kpos >= k_lo && kpos <= qpos_last) {
        const size_t off = kv_offset_of(table, kpos, kvh, a) + (size_t)c * VEC;
        Vec<T> kv, vv;
        kv.load(kc + off);
        vv.load(vc + off);
        kv.unpack(kf);
        vv.unpack(vf);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) { kf[e] = 0.f; vf[e] = 0.f; }
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        Ks[kk * DS + c * VEC + e] = kf[e];
        Vs[kk * D + c * VEC + e] = vf[e];
      }
    }
    __syncthreads();
    // ---- scores: thread (ty, tx) owns rows ty*4..+3, keys tx*2..+1
    float s[4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i) { s[i][0] = 0.f; s[i][1] = 0.f; }
    for (int d = 0; d < D; ++d) {
      const float kv0 = Ks[(tx * 2) * DS + d], kv1 = Ks[(tx * 2 + 1) * DS + d];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float qv = Qs[(ty * 4 + i) * DS + d];
        s[i][0] = fmaf(qv, kv0, s[i][0]);
        s[i][1] = fmaf(qv, kv1, s[i][1]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty * 4 + i;
      const int qpos = first_pos + q0 + r;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int kpos = k0 + tx * 2 + j;
        bool ok = (r < nq) && (kpos <= qpos);
        if (a.window > 0) ok = ok && (kpos > qpos - a.window);
        Ss[r * (PF_TK + 1) + tx * 2 + j] = ok ? s[i][j] : NEG_INF;
      }
    }
    __syncthreads();
    // ---- online softmax per row: 4 threads per row
    {
      const int r = tid >> 2, part = tid & 3;
      float* srow = Ss + r * (PF_TK + 1);
      float mx = NEG_INF;
#pragma unroll
      for (int j = 0; j < PF_TK / 4; ++j) mx = fmaxf(mx, srow[part * (PF_TK / 4) + j]);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_old = row_m[r];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < PF_TK / 4; ++j) {
        const int col = part * (PF_TK / 4) + j;
        const float sv = srow[col];
        const float p = (sv == NEG_INF) ? 0.f : exp2f(sv - m_new);
        srow[col] = p;
        sum += p;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      __syncwarp();
      if (part == 0) {
        const float corr = (m_new == NEG_INF) ? 1.f : exp2f(m_old - m_new);  // m_old = -inf gives 0
        row_c[r] = corr;
        row_l[r] = row_l[r] * corr + sum;
        row_m[r] = m_new;
      }
    }
    __syncthreads();
    // ---- acc = acc * corr + P V: thread owns rows ty*4..+3, columns tx + 16 j
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float corr = row_c[ty * 4 + i];
#pragma unroll
      for (int j = 0; j < DJMAX; ++j) acc[i][j] *= corr;
    }
    for (int kk = 0; kk < PF_TK; ++kk) {
      float p[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) p[i] = Ss[(ty * 4 + i) * (PF_TK + 1) + kk];
#pragma unroll
      for (int j = 0; j < DJMAX; ++j) {
        if (j < dj) {
          const float vv = Vs[kk * D + tx + 16 * j];
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i][j] = fmaf(p[i], vv, acc[i][j]);
        }
      }
    }
  }
  __syncthreads();
  T* out = (T*)a.out;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r < nq) {
      const float inv = 1.f / row_l[r];
#pragma unroll
      for (int j = 0; j < DJMAX; ++j)
        if (j < dj)
          out[((size_t)(row0 + q0 + r) * a.num_heads + head) * D + tx + 16 * j] = from_float<T>(acc[i][j] * inv);
    }
  }
}

// ================================================================ decode (split-K)
constexpr int DC_WARPS = 4;
constexpr int DC_THREADS = DC_WARPS * 32;
constexpr int DC_MAX_COUNTERS = 1 << 16;

// One arrival counter per (request, CTA row of the grid): the CTA that arrives last merges the
// key ranges. Counters are zero when the library is loaded and every merge puts its counter
// back to zero, so no launch ever has to clear them.
static __device__ unsigned int g_decode_counters[DC_MAX_COUNTERS];

// GT = query heads handled per CTA (a kv group is covered by ceil(G / GT) CTAs);
// CPL = 16-byte chunks of a key per lane; U = keys per lane group whose loads are in flight.
template <typename T, int GT, int CPL, int U>
__global__ void __launch_bounds__(DC_THREADS) decode_attn_kernel(AttnArgs a, int lanes_per_key, int passes) {
  constexpr int VEC = Vec<T>::N;
  constexpr int EPL = VEC * CPL;                 // elements of a key per lane
  extern __shared__ float smem[];                // [DC_WARPS][GT][D + 2]
  __shared__ int is_last;
  pdl_trigger();
  const int D = a.head_dim;
  const int G = a.num_heads / a.num_kv_heads;
  const int si = blockIdx.x;
  const int kvh = blockIdx.y / passes;
  const int g0 = (blockIdx.y - kvh * passes) * GT;   // first head of the group this CTA handles
  const int ng = min(GT, G - g0);
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int LPK = lanes_per_key;
  const int sub = lane / LPK, lk = lane - sub * LPK;  // which key of the warp's batch, which lane of it
  const int KPW = 32 / LPK;                           // keys per warp per batch
  const int chunks = D / VEC;
  pdl_wait();

  const int seq = a.seq_ids[si];
  const int ctx = a.ctx_lens[seq];
  const int qrow = a.cu_q[seq];
  const int lo = (a.window > 0) ? max(0, ctx - a.window) : 0;
  const int len = ctx - lo;
  const int per = (len + a.num_splits - 1) / a.num_splits;
  const int k_begin = lo + split * per;
  const int k_end = min(ctx, k_begin + per);
  const int* table = a.block_tables + (size_t)seq * a.table_width;
  const T* kc = (const T*)a.k_cache;
  const T* vc = (const T*)a.v_cache;

  // this lane's share of every query head, pre-scaled
  float qreg[GT][EPL];
#pragma unroll
  for (int g = 0; g < GT; ++g)
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
      const int chunk = lk + c * LPK;
      float f[VEC];
      if (g < ng && chunk < chunks) {
        Vec<T> v;
        v.load((const T*)a.q + ((size_t)qrow * a.num_heads + kvh * G + g0 + g) * D + chunk * VEC);
        v.unpack(f);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) f[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) qreg[g][c * VEC + e] = f[e] * a.scale_log2;
    }

  float m[GT], l[GT], acc[GT][EPL];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = NEG_INF;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
  }

  const int stride = DC_WARPS * KPW * U;
  for (int base = k_begin + (warp * U) * KPW; base < k_end; base += stride) {
    // ---- all loads of this batch first: U keys and U values per lane group, kept packed
    Vec<T> kraw[U][CPL], vraw[U][CPL];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kpos = base + u * KPW + sub;
      valid[u] = kpos < k_end;
      size_t off = 0;
      if (valid[u]) off = kv_offset_of(table, kpos, kvh, a);
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const int chunk = lk + c * LPK;
        if (valid[u] && chunk < chunks) {
          kraw[u][c].load(kc + off + (size_t)chunk * VEC);
          vraw[u][c].load(vc + off + (size_t)chunk * VEC);
        } else {
          kraw[u][c].zero();
          vraw[u][c].zero();
        }
      }
    }
    // ---- scores
    float s[GT][U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float kf[EPL];
#pragma unroll
      for (int c = 0; c < CPL; ++c) kraw[u][c].unpack(&kf[c * VEC]);
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) d = fmaf(qreg[g][e], kf[e], d);
        s[g][u] = d;
      }
    }
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float d = s[g][u];
        for (int o = LPK >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        s[g][u] = valid[u] ? d : NEG_INF;
      }
    // ---- online softmax, one rescale per batch
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float m_new = m[g];
#pragma unroll
      for (int u = 0; u < U; ++u) m_new = fmaxf(m_new, s[g][u]);
      const float corr = (m_new == NEG_INF) ? 1.f : exp2f(m[g] - m_new);   // m = -inf gives 0
      float psum = 0.f;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float p = (s[g][u] == NEG_INF) ? 0.f : exp2f(s[g][u] - m_new);
        s[g][u] = p;
        psum += p;
      }
      l[g] = l[g] * corr + psum;
      m[g] = m_new;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc[g][e] *= corr;
    }
    // ---- values
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float vf[EPL];
#pragma unroll
      for (int c = 0; c < CPL; ++c) vraw[u][c].unpack(&vf[c * VEC]);
#pragma unroll
      for (int g = 0; g < GT; ++g)
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = fmaf(s[g][u], vf[e], acc[g][e]);
    }
  }

  // ---- merge the lane groups of a warp (lanes with equal lk hold the same elements)
  for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m[g], o);
      const float l2 = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float mn = fmaxf(m[g], m2);
      const float c1 = (mn == NEG_INF) ? 1.f : exp2f(m[g] - mn);
      const float c2 = (mn == NEG_INF) ? 1.f : exp2f(m2 - mn);
      l[g] = l[g] * c1 + l2 * c2;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float a2 = __shfl_xor_sync(0xffffffffu, acc[g][e], o);
        acc[g][e] = acc[g][e] * c1 + a2 * c2;
      }
      m[g] = mn;
    }
  }
  // ---- merge the warps through shared memory
  const int WS = D + 2;
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float* w = smem + ((size_t)warp * GT + g) * WS;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const int chunk = lk + c * LPK;
        if (chunk < chunks)
#pragma unroll
          for (int e = 0; e < VEC; ++e) w[chunk * VEC + e] = acc[g][c * VEC + e];
      }
      if (lk == 0) { w[D] = m[g]; w[D + 1] = l[g]; }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < ng * D; idx += DC_THREADS) {
    const int g = idx / D, d = idx - g * D;
    float mm = NEG_INF;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) mm = fmaxf(mm, smem[((size_t)w * GT + g) * WS + D]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) {
      const float* ws = smem + ((size_t)w * GT + g) * WS;
      const float c = (ws[D] == NEG_INF) ? 0.f : exp2f(ws[D] - mm);
      num += ws[d] * c;
      den += ws[D + 1] * c;
    }
    const int head = kvh * G + g0 + g;
    if (a.num_splits == 1) {
      ((T*)a.out)[((size_t)qrow * a.num_heads + head) * D + d] = from_float<T>(num / den);
    } else {
      const size_t pidx = ((size_t)si * a.num_heads + head) * a.num_splits + split;
      a.part_acc[pidx * D + d] = num;
      if (d == 0) { a.part_ml[pidx * 2] = mm; a.part_ml[pidx * 2 + 1] = den; }
    }
  }
  if (a.num_splits == 1) return;

  // ---- the CTA that arrives last for this (request, heads) merges the ranges
  unsigned int* counter = &g_decode_counters[((size_t)si * gridDim.y + blockIdx.y) % DC_MAX_COUNTERS];
  if (!cta_arrives_last(counter, (unsigned int)a.num_splits, &is_last)) return;
  merge_splits<T>(a, si, qrow, kvh * G + g0, ng, smem);
}

template <typename T, int DJMAX>
static int launch_prefill_dj(const AttnArgs& a, int max_query_len, cudaStream_t stream) {
  const int D = a.head_dim;
  const size_t smem = sizeof(float) * ((size_t)PF_TQ * (D + 1) + (size_t)PF_TK * (D + 1) + (size_t)PF_TK * D +
                                       (size_t)PF_TQ * (PF_TK + 1) + 3 * PF_TQ);
  auto kern = prefill_attn_kernel<T, DJMAX>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((max_query_len + PF_TQ - 1) / PF_TQ, a.num_seqs, a.num_heads);
  return launch(kern, grid, PF_THREADS, smem, stream, a);
}

template <typename T>
static int launch_prefill(const AttnArgs& a, int max_query_len, cudaStream_t stream) {
  const int dj = a.head_dim / 16;
  if (dj <= 2) return launch_prefill_dj<T, 2>(a, max_query_len, stream);
  if (dj <= 4) return launch_prefill_dj<T, 4>(a, max_query_len, stream);
  if (dj <= 8) return launch_prefill_dj<T, 8>(a, max_query_len, stream);
  return launch_prefill_dj<T, 16>(a, max_query_len, stream);
}

template <typename T, int GT, int CPL>
static int launch_decode_gc(const AttnArgs& a, int lpk, cudaStream_t stream) {
  constexpr int U = (CPL == 1 && GT <= 4) ? 8 : 4;
  const int G = a.num_heads / a.num_kv_heads;
  const int passes = (G + GT - 1) / GT;
  if ((long long)a.num_seqs * a.num_kv_heads * passes > DC_MAX_COUNTERS && a.num_splits > 1) return TS_ERR_UNSUPPORTED;
  const size_t smem = sizeof(float) * (size_t)DC_WARPS * GT * (a.head_dim + 2);
  auto kern = decode_attn_kernel<T, GT, CPL, U>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(a.num_seqs, a.num_kv_heads * passes, a.num_splits);
  return launch(kern, grid, DC_THREADS, smem, stream, a, lpk, passes);
}

template <typename T>
static int launch_decode(const AttnArgs& a, cudaStream_t stream) {
  constexpr int VEC = Vec<T>::N;
  const int chunks = a.head_dim / VEC;
  int lpk = 1;
  while (lpk < chunks && lpk < 32) lpk <<= 1;
  const int cpl = (chunks + lpk - 1) / lpk;
  const int G = a.num_heads / a.num_kv_heads;
  if (cpl > 2) return TS_ERR_UNSUPPORTED;
#define TS_DECODE_CASE(GT_)                                                   \
  return cpl == 1 ? launch_decode_gc<T, GT_, 1>(a, lpk, stream) : launch_decode_gc<T, GT_, 2>(a, lpk, stream)
  if (G == 1) { TS_DECODE_CASE(1); }
  if (G == 2) { TS_DECODE_CASE(2); }
  if (G <= 4) { TS_DECODE_CASE(4); }
  TS_DECODE_CASE(8);
#undef TS_DECODE_CASE
}

}  // namespace ts

