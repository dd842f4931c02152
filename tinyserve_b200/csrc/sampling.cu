// Next-token selection on the device: greedy argmax, temperature sampling, nucleus (top-p).
//
// Meaning of the options follows upstream src/tinyserve/sampling.py:56-102: temperature 0 is
// the argmax of the raw 32-bit logits; otherwise the token is drawn from softmax(logits / T)
// by the exponential race argmax_i p_i / E_i with E_i ~ Exp(1); with top_p < 1 only tokens are
// eligible whose more likely tokens together hold less than top_p of the mass (the most likely
// token always is), without renormalising. Differences: the noise comes from a counter-based
// generator (Philox4x32-10) keyed by the request's seed and indexed by (how many tokens the
// request has drawn, token id), so a request's tokens do not depend on its batch-mates, on
// chunking or on recomputation; tokens of exactly equal probability are kept or dropped
// together by top-p; the race is run on logit / T - log E_i, which orders the same way.
//
// A row without top-p is cut into chunks, one CTA each; the CTA that arrives last picks the
// winner among the chunks' winners. A row with top-p needs sums over the whole row and is done
// by one CTA.
#define TS_PDL_CLASS PDL_SAMPLING
#include "common.cuh"

namespace ts {

constexpr int SM_THREADS = 1024;
constexpr int SM_MAX_ROWS = 4096;
constexpr int SM_MAX_CHUNKS = 32;

struct Best {
  float v;
  int i;
};
// Winners of the chunks, and an arrival counter per row that the last CTA puts back to zero.
static __device__ Best g_chunk_best[SM_MAX_ROWS * SM_MAX_CHUNKS];
static __device__ unsigned int g_row_arrivals[SM_MAX_ROWS];

__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.i < 0) return a;
  if (a.i < 0) return b;
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ Best block_best(Best x, Best* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  Best t;
  t.v = 0.f; t.i = -1;
  if (lane < nwarps) t = scratch[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, t.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, t.i, o);
    t = better(t, y);
  }
  return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
  return warp_max(t);
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t out[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// exp(logit / T - max) with each step rounded on its own, so that the nucleus threshold found by
// the search and the later eligibility test see bit-identical values (no fused multiply-add).
__device__ __forceinline__ float scaled(float logit, float inv_t) { return __fmul_rn(logit, inv_t); }
__device__ __forceinline__ float weight_of(float logit, float inv_t, float mx) {
  return expf(__fsub_rn(scaled(logit, inv_t), mx));
}

// -log(u) with u uniform in (0, 1) on a 24-bit grid: never 0, never infinite.
__device__ __forceinline__ float exp1_from_bits(uint32_t x) {
  const float u = ((float)(x >> 8) + 0.5f) * (1.0f / 16777216.0f);
  return -logf(u);
}

// Best candidate of tokens [begin, end) (begin a multiple of 4) for one row.
// threshold: tokens with exp(z - mx) below it are not eligible (0 = all are).
__device__ __forceinline__ Best scan_range(const float* __restrict__ l, int begin, int end, float temp,
                                           float mx, float threshold, uint32_t k0, uint32_t k1, uint32_t d0,
                                           uint32_t d1) {
  Best best;
  best.v = 0.f; best.i = -1;
  if (!(temp > 0.f)) {
    // greedy: a thread's indices only grow, so "strictly greater" keeps the first maximum.
    float bv = -INFINITY;
    int bi = -1;
    if ((((uintptr_t)l) & 15) == 0) {
      const float4* l4 = reinterpret_cast<const float4*>(l);
      for (int i4 = begin / 4 + threadIdx.x; i4 * 4 < end; i4 += blockDim.x) {
        const int i = i4 * 4;
        if (i + 4 <= end) {
          const float4 v = l4[i4];
          if (v.x > bv) { bv = v.x; bi = i; }
          if (v.y > bv) { bv = v.y; bi = i + 1; }
          if (v.z > bv) { bv = v.z; bi = i + 2; }
          if (v.w > bv) { bv = v.w; bi = i + 3; }
        } else {
          for (int e = i; e < end; ++e)
            if (l[e] > bv) { bv = l[e]; bi = e; }
        }
      }
    } else {
      for (int i = begin + threadIdx.x; i < end; i += blockDim.x)
        if (l[i] > bv) { bv = l[i]; bi = i; }
    }
    if (bi < 0 && begin + (int)threadIdx.x < end) { bv = l[begin + threadIdx.x]; bi = begin + threadIdx.x; }  // all -inf / NaN
    best.v = bv; best.i = bi;
    return best;
  }
  const float inv_t = 1.f / temp;
  for (int i4 = begin / 4 + threadIdx.x; i4 * 4 < end; i4 += blockDim.x) {
    uint32_t r[4];
    philox4x32_10((uint32_t)i4, d0, d1, 0u, k0, k1, r);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = i4 * 4 + e;
      if (i < end) {
        const float z = scaled(l[i], inv_t);
        if (threshold <= 0.f || weight_of(l[i], inv_t, mx) >= threshold) {
          Best c; c.v = z - logf(exp1_from_bits(r[e])); c.i = i;
          best = better(best, c);
        }
      }
    }
  }
  return best;
}

__global__ void __launch_bounds__(SM_THREADS) sample_kernel(const float* __restrict__ logits, int vocab,
                                                            const float* __restrict__ temperature,
                                                            const float* __restrict__ top_p,
                                                            const long long* __restrict__ seeds,
                                                            const long long* __restrict__ draws,
                                                            int* __restrict__ out, int chunks,
                                                            const int* __restrict__ status_in,
                                                            int* __restrict__ status_out) {
  __shared__ float fscratch[33];
  __shared__ Best bscratch[32];
  __shared__ int is_last;
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x, chunk = blockIdx.y;
  // the step's error word (set by a kernel whose bounded wait ran out) travels to the host with the tokens
  if (status_out != nullptr && row == 0 && chunk == 0 && threadIdx.x == 0) *status_out = status_in ? *status_in : 0;
  const float* l = logits + (size_t)row * vocab;
  const float temp = temperature ? temperature[row] : 0.f;
  const float tp = (top_p && temp > 0.f) ? top_p[row] : 1.f;
  uint32_t k0 = 0, k1 = 0, d0 = 0, d1 = 0;
  if (temp > 0.f) {
    k0 = (uint32_t)(seeds[row] & 0xffffffffll); k1 = (uint32_t)((unsigned long long)seeds[row] >> 32);
    d0 = (uint32_t)(draws[row] & 0xffffffffll); d1 = (uint32_t)((unsigned long long)draws[row] >> 32);
  }

  if (tp < 1.f) {
    // ---- nucleus: the whole row in the CTA of chunk 0
    if (chunk != 0) return;
    const float inv_t = 1.f / temp;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, scaled(l[i], inv_t));
    mx = block_max(mx, fscratch);
    float z = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) z += weight_of(l[i], inv_t, mx);
    z = block_sum(z, fscratch);
    const float target = tp * z;
    // smallest bit pattern b in [0, bits(1.0)] with mass{e > float(b)} < target
    uint32_t lo = 0u, hi = 0x3f800000u;
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1);
      const float t = __uint_as_float(mid);
      float mass = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float e = weight_of(l[i], inv_t, mx);
        if (e > t) mass += e;
      }
      mass = block_sum(mass, fscratch);
      if (mass < target) hi = mid; else lo = mid + 1u;
    }
    Best best = scan_range(l, 0, vocab, temp, mx, __uint_as_float(lo), k0, k1, d0, d1);
    best = block_best(best, bscratch);
    if (threadIdx.x == 0) out[row] = best.i < 0 ? 0 : best.i;
    return;
  }

  // ---- greedy or temperature only: this CTA's chunk, then the last CTA picks among chunks
  int per = (vocab + chunks - 1) / chunks;
  per = (per + 3) & ~3;
  const int begin = chunk * per, end = min(vocab, begin + per);
  Best best = scan_range(l, begin, end, temp, 0.f, 0.f, k0, k1, d0, d1);
  best = block_best(best, bscratch);
  if (chunks == 1) {
    if (threadIdx.x == 0) out[row] = best.i < 0 ? 0 : best.i;
    return;
  }
  if (threadIdx.x == 0) g_chunk_best[row * SM_MAX_CHUNKS + chunk] = best;
  if (!cta_arrives_last(&g_row_arrivals[row], (unsigned int)chunks, &is_last)) return;
  if (threadIdx.x < 32) {
    // one lane per chunk (chunks <= 32): independent loads, then a warp reduction
    Best b;
    b.v = 0.f; b.i = -1;
    if ((int)threadIdx.x < chunks) {
      b.v = __ldcg(&g_chunk_best[row * SM_MAX_CHUNKS + threadIdx.x].v);
      b.i = __ldcg(&g_chunk_best[row * SM_MAX_CHUNKS + threadIdx.x].i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best y;
      y.v = __shfl_xor_sync(0xffffffffu, b.v, o);
      y.i = __shfl_xor_sync(0xffffffffu, b.i, o);
      b = better(b, y);
    }
    if (threadIdx.x == 0) out[row] = b.i < 0 ? 0 : b.i;
  }
}

}  // namespace ts

using namespace ts;

// temperature/top_p/seeds/draws may all be null for an all-greedy batch. status_out (optional)
// receives *status_in (0 if that is null): the device word that kernels with bounded waits set
// when a wait ran out, so that one copy brings the tokens and the step's status to the host.
extern "C" int ts_sample(const float* logits, int num_rows, int vocab, const float* temperature,
                         const float* top_p, const long long* seeds, const long long* draws, int* out,
                         const int* status_in, int* status_out, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (vocab <= 0 || num_rows > SM_MAX_ROWS) return TS_ERR_BAD_ARGUMENT;
  if (temperature != nullptr && (seeds == nullptr || draws == nullptr)) return TS_ERR_BAD_ARGUMENT;
  // as many CTAs as run at once (two of 1024 threads per SM), never a partly filled second
  // round, each with at least a few thousand tokens
  int chunks = (148 * 2) / num_rows;
  const int most = (vocab + 4095) / 4096;
  if (chunks > most) chunks = most;
  if (chunks > SM_MAX_CHUNKS) chunks = SM_MAX_CHUNKS;
  if (chunks < 1) chunks = 1;
  return launch(sample_kernel, dim3(num_rows, chunks), SM_THREADS, 0, stream, logits, vocab, temperature, top_p,
                seeds, draws, out, chunks, status_in, status_out);
}
