// out[M, N] = x[M, K] * w[N, K]^T for a handful of rows (decode: M = live requests), bf16 in,
// 32-bit accumulation on the tensor cores, bf16 or float out; optionally the SwiGLU product
// out[m, j] = silu(x w[j]) * (x w[N + j]) of a merged gate/up matrix in the same pass.
//
// The product is memory-bound: every weight is read once and used M times. So the weights are
// the A operand (16 weight rows per mma tile), streamed straight from global memory into the
// mma fragments with 16-byte loads that never pass through shared memory, and the few rows of x
// are the B operand (8 columns per tile), read through L1. Each lane loads 8 consecutive k of
// "its" weight row and of "its" x row; which k feeds which slot of the mma does not matter as
// long as A and B agree, so those 8 values serve two m16n8k16 instructions without any shuffle.
// A CTA owns 16 * RT weight rows (twice that when fused); its 8 warps split K between them and
// add their partial sums in shared memory in a fixed order, so the result is deterministic.
// The first weight loads are issued before the kernel waits for its predecessor (weights do not
// depend on it), so under programmatic dependent launch the weights of one product stream in
// while the previous kernel is still finishing.
//
// When the matrix has too few rows to give every SM work (N / 16 CTAs), K is also split across
// CTAs (grid.y): each writes its partial sums to a scratch array of the library, and the CTA of
// a row tile that arrives last adds the parts in slice order (deterministic) and writes the
// result. The scratch and the arrival counters are fixed arrays of the library, so products on
// different streams must not overlap.
//
// Two optional fusions with the RMSNorm around the product (decode steps, where a norm kernel of
// its own costs more than its work):
//  * NORMX: x is not given; the kernel forms it from a bf16 copy r16 of the residual stream
//    and the norm weight as bf16(r16 * weight), and scales the finished sums by the row's rstd =
//    rsqrt(mean(r^2) + eps) in 32-bit (the norm of upstream src/tinyserve/layers.py:35-38; the
//    scale is a factor of the whole row, so it commutes with the product). The sums of squares
//    (of the 32-bit stream) come in parts from the producer of the stream and are added in a
//    fixed order, off the critical path. The copy is bf16 because every CTA reads all of it from
//    L2: a 32-bit read was measured to cost more than the norm kernel it saves.
//  * RESID: the result is not stored; rounded to bf16 it is added to the residual stream in
//    place, and the bf16 copy of the new stream and the sum of its squares over this CTA's 16
//    columns are written per row for the next NORMX consumer.
//
// Needs K % 32 == 0 and N % 16 == 0 (the launcher reports TS_ERR_UNSUPPORTED otherwise and the
// caller takes another kernel).
#define TS_PDL_CLASS PDL_SKINNY
#include "common.cuh"

namespace ts {

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_KSTEP = SK_WARPS * 32;    // distance between a warp's k blocks
constexpr int SK_MAX_SPLIT = 8;
constexpr int SK_TALL_WARPS = 16, SK_TALL_PF = 6;
constexpr int SK_SPLIT_MAX_ROWS = 16;      // K is split across CTAs only for M up to this
constexpr int SK_SPLIT_MAX_COLS = 2 * 6144;   // and for at most this many (gate + up) columns
constexpr int SK_MAX_TILES = 1024;

// Partial sums [slice][m][column] of the products whose K is split across CTAs, and one
// arrival counter per row tile, which the last CTA puts back to zero.
static __device__ float g_skinny_partial[SK_MAX_SPLIT * SK_SPLIT_MAX_ROWS * SK_SPLIT_MAX_COLS];
static __device__ unsigned int g_skinny_arrivals[SK_MAX_TILES];

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cached(const void* p) {
  uint4 v;
  asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT = column tiles of 8 rows of x (M <= 8 * NT); RT = weight row tiles of 16 per CTA (each x
// fragment is used for all of them); SK_PF = k blocks of a warp whose weights are in flight;
// FUSE: w holds 2 N rows (gate rows, then up rows) and out = silu(gate) * up, [M, N].
struct SkinnyNorm {
  const bf16* resid16;    // NORMX: [M, K] bf16 copy of the residual stream
  const float* sumsq;     // NORMX: [M][parts] partial sums of squares of the rows of the stream
  int parts;
  const bf16* weight;     // NORMX: [K] norm weight
  float eps;
  float* resid_out;       // RESID: [M, N] the 32-bit stream, added to in place
  bf16* resid16_out;      // RESID: [M, N] its bf16 copy
  float* sumsq_out;       // RESID: [M][N / 16]
};

__device__ __forceinline__ uint4 ld_cg(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
// bf16(r16 * weight) for 8 consecutive k: the B fragment of a NORMX product.
__device__ __forceinline__ uint4 normed_fragment(const uint4& rv, const uint4& wv) {
  const uint32_t rr[4] = {rv.x, rv.y, rv.z, rv.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float r0 = __uint_as_float(rr[i] << 16), r1 = __uint_as_float(rr[i] & 0xffff0000u);
    const float w0 = __uint_as_float(ww[i] << 16), w1 = __uint_as_float(ww[i] & 0xffff0000u);
    __nv_bfloat162 h = __floats2bfloat162_rn(r0 * w0, r1 * w1);
    o[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// WARPS: warps of a CTA, which split K between them (8; 16 in the tall form, see launch_skinny).
// The forms of up to 16 rows are held to 128 registers so that two CTAs of 8 warps fit an SM: the
// fused gate/up product of 9 to 16 rows took 146 and ran its 192 CTAs in two rounds (10.4 us in a
// recorded decode step of 16 rows, against 6.6 us for the 8-row form).
template <typename TOut, int NT, int RT, bool FUSE, int SK_PF, bool XRING, bool NORMX = false, bool RESID = false,
          int WARPS = SK_WARPS>
__global__ void __launch_bounds__(WARPS * 32, (WARPS == 8 && NT <= 2) ? 2 : 1)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                                 TOut* __restrict__ out, int M, int N, int K,
                                                                 SkinnyNorm nrm) {
  static_assert(!(RESID && FUSE), "the fused activation is not added to the stream");
  static_assert(!NORMX || WARPS == 8, "the sums of squares are spread over eight warps");
  constexpr int KSTEP = WARPS * 32;      // distance between a warp's k blocks
  constexpr int TILES = FUSE ? 2 * RT : RT;
  constexpr int COLS = 8 * NT;
  // a row of partial sums is COLS + 1 long: the threads that add them up take consecutive rows, which
  // would otherwise fall into two or four banks (16- and 8-fold conflicts on every read)
  constexpr int CS = COLS + 1;
  extern __shared__ float red[];   // [WARPS][TILES][16][CS]
  __shared__ int is_last;
  __shared__ float rstd_s[16];
  pdl_trigger();
  // this CTA's slice of K (the whole of it unless grid.y > 1)
  const int ksplit = gridDim.y;
  const int k_len = K / ksplit;
  const int k_lo = blockIdx.y * k_len, k_hi = k_lo + k_len;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * (16 * RT);

  const bf16* wrow[TILES][2];
#pragma unroll
  for (int r = 0; r < TILES; ++r) {
    const int base = (r < RT) ? n0 + r * 16 : N + n0 + (r - RT) * 16;
    wrow[r][0] = w + (size_t)(base + g) * K + 8 * t;
    wrow[r][1] = w + (size_t)(base + g + 8) * K + 8 * t;
  }
  // weights of the first SK_PF k blocks of this warp: in flight before the predecessor is done
  uint4 ring[SK_PF][TILES][2];
#pragma unroll
  for (int p = 0; p < SK_PF; ++p) {
    const int kb = k_lo + warp * 32 + p * KSTEP;
    if (kb < k_hi) {
#pragma unroll
      for (int r = 0; r < TILES; ++r) {
        ring[p][r][0] = ld_stream(wrow[r][0] + kb);
        ring[p][r][1] = ld_stream(wrow[r][1] + kb);
      }
    }
  }
  pdl_wait();
  // RESID: the value of the stream that this thread will add to, fetched now instead of at the end (the
  // epilogue's loop runs once per thread, and the trip to L2 was 700 of the kernel's 9,500 cycles)
  float resid_before = 0.f;
  if constexpr (RESID) {
    static_assert(RT * 16 * 8 * NT <= WARPS * 32, "one output per thread");
    const int idx = threadIdx.x, m = idx / (RT * 16), row = idx - m * (RT * 16);
    if (gridDim.y == 1 && idx < RT * 16 * 8 * NT && m < M) resid_before = ld_cg_f32(nrm.resid_out + (size_t)m * N + n0 + row);
  }

  float acc[TILES][NT][4];
#pragma unroll
  for (int r = 0; r < TILES; ++r)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[r][j][e] = 0.f;
  const bf16* xrow[NT];
  const bf16* rrow[NT];
  bool xok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int m = 8 * j + g;
    xok[j] = m < M;
    xrow[j] = x + (size_t)(xok[j] ? m : 0) * K + 8 * t;
    rrow[j] = NORMX ? nrm.resid16 + (size_t)(xok[j] ? m : 0) * K + 8 * t : nullptr;
  }
  // NORMX: the parts of the rows' sums of squares are fetched now and added when the products are
  // done (nothing waits for them meanwhile): warp w takes rows w and w + 8, a lane up to four parts
  float ssq[2][4];
  if constexpr (NORMX) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = warp + 8 * h, p = lane + 32 * i;
        ssq[h][i] = (m < M && p < nrm.parts) ? ld_cg_f32(nrm.sumsq + m * nrm.parts + p) : 0.f;
      }
  }
  // XRING: the fragments of x are fetched as far ahead as the weights. Chosen when a warp has so
  // few k blocks that all its loads go out at once and nothing later waits for L2; with long
  // loops the extra registers would cost more in occupancy than the prefetch gains.
  uint4 xring[XRING ? SK_PF : 1][NT];
  uint4 wring[(XRING && NORMX) ? SK_PF : 1];      // NORMX: the norm weight of the same k, converted at use
  if constexpr (XRING) {
#pragma unroll
    for (int p = 0; p < SK_PF; ++p) {
      const int kb = k_lo + warp * 32 + p * KSTEP;
#pragma unroll
      for (int j = 0; j < NT; ++j)
        xring[p][j] = !(kb < k_hi && xok[j]) ? make_uint4(0u, 0u, 0u, 0u) : ld_cached((NORMX ? rrow[j] : xrow[j]) + kb);
      if constexpr (NORMX) wring[p] = kb < k_hi ? ld_cached(nrm.weight + kb + 8 * t) : make_uint4(0u, 0u, 0u, 0u);
    }
  }

  for (int kb0 = k_lo + warp * 32; kb0 < k_hi; kb0 += SK_PF * KSTEP) {
#pragma unroll
    for (int p = 0; p < SK_PF; ++p) {
      const int kb = kb0 + p * KSTEP;
      if (kb < k_hi) {
        uint4 a[TILES][2];
#pragma unroll
        for (int r = 0; r < TILES; ++r) { a[r][0] = ring[p][r][0]; a[r][1] = ring[p][r][1]; }
        uint4 b[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          if constexpr (XRING && NORMX) b[j] = normed_fragment(xring[p][j], wring[p]);
          else if constexpr (XRING) b[j] = xring[p][j];
          else if constexpr (NORMX) b[j] = xok[j] ? normed_fragment(ld_cached(rrow[j] + kb), ld_cached(nrm.weight + kb + 8 * t)) : make_uint4(0u, 0u, 0u, 0u);
          else b[j] = xok[j] ? ld_cached(xrow[j] + kb) : make_uint4(0u, 0u, 0u, 0u);
        }
        const int nxt = kb + SK_PF * KSTEP;
        if (nxt < k_hi) {
#pragma unroll
          for (int r = 0; r < TILES; ++r) {
            ring[p][r][0] = ld_stream(wrow[r][0] + nxt);
            ring[p][r][1] = ld_stream(wrow[r][1] + nxt);
          }
          if constexpr (XRING) {
#pragma unroll
            for (int j = 0; j < NT; ++j) xring[p][j] = xok[j] ? ld_cached((NORMX ? rrow[j] : xrow[j]) + nxt) : make_uint4(0u, 0u, 0u, 0u);
            if constexpr (NORMX) wring[p] = ld_cached(nrm.weight + nxt + 8 * t);
          }
        }
#pragma unroll
        for (int r = 0; r < TILES; ++r)
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            mma_bf16_16816(acc[r][j], a[r][0].x, a[r][1].x, a[r][0].y, a[r][1].y, b[j].x, b[j].y);
            mma_bf16_16816(acc[r][j], a[r][0].z, a[r][1].z, a[r][0].w, a[r][1].w, b[j].z, b[j].w);
          }
      }
    }
  }

  if constexpr (NORMX) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = warp + 8 * h;
      const float ss = warp_sum((ssq[h][0] + ssq[h][1]) + (ssq[h][2] + ssq[h][3]));      // a fixed order
      if (lane == 0 && m < M) rstd_s[m] = rsqrtf(ss / (float)K + nrm.eps);
    }
  }
  // partial sums of this warp -> shared memory; element (row, col) of tile (r, j)
  float* mine = red + (size_t)warp * TILES * 16 * CS;
#pragma unroll
  for (int r = 0; r < TILES; ++r)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      float* tile = mine + (size_t)r * 16 * CS + j * 8;
      tile[g * CS + 2 * t] = acc[r][j][0];
      tile[g * CS + 2 * t + 1] = acc[r][j][1];
      tile[(g + 8) * CS + 2 * t] = acc[r][j][2];
      tile[(g + 8) * CS + 2 * t + 1] = acc[r][j][3];
    }
  __syncthreads();
  // thread -> (column m, weight row): consecutive threads take consecutive weight rows, so a
  // column of the result is written as one run of out[m, n0 .. n0 + 16 RT).
  const int width = FUSE ? 2 * N : N;                 // columns of a partial row
  float* part = g_skinny_partial + (size_t)blockIdx.y * SK_SPLIT_MAX_ROWS * width;
  // RESID: add to the stream and leave the row's sum of squares over these 16 columns (RT = 1:
  // the 16 threads of a row are half a warp; every lane of the warp takes part in the shuffles)
  auto to_stream = [&](int m, int row, float s, bool fetched) {
    float r = 0.f;
    if (m < M) {
      float* rp = nrm.resid_out + (size_t)m * N + n0 + row;
      r = (fetched ? resid_before : *rp) + round_to<bf16>(s);
      *rp = r;
      nrm.resid16_out[(size_t)m * N + n0 + row] = from_float<bf16>(r);
    }
    float sq = r * r;
    sq += __shfl_xor_sync(0xffffffffu, sq, 8);
    sq += __shfl_xor_sync(0xffffffffu, sq, 4);
    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
    if (row == 0 && m < M) nrm.sumsq_out[m * gridDim.x + blockIdx.x] = sq;
  };
  for (int idx = threadIdx.x; idx < RT * 16 * COLS; idx += WARPS * 32) {
    const int m = idx / (RT * 16), row = idx - m * (RT * 16);
    float s = 0.f, u = 0.f;
    if (m < M) {
#pragma unroll
      for (int wq = 0; wq < WARPS; ++wq) s += red[(size_t)wq * TILES * 16 * CS + row * CS + m];
      if constexpr (FUSE) {
#pragma unroll
        for (int wq = 0; wq < WARPS; ++wq) u += red[(size_t)wq * TILES * 16 * CS + (RT * 16 + row) * CS + m];
      }
      if (ksplit > 1) {
        part[(size_t)m * width + n0 + row] = s;
        if constexpr (FUSE) part[(size_t)m * width + N + n0 + row] = u;
      } else if constexpr (NORMX) {
        s *= rstd_s[m];
        u *= rstd_s[m];
      }
      if (ksplit > 1) {
      } else if constexpr (FUSE) {
        // rounding points of the unfused path: product -> bf16, silu -> bf16, times up -> bf16
        const float gv = round_to<bf16>(s), uv = round_to<bf16>(u);
        const float sv = round_to<bf16>(gv / (1.f + expf(-gv)));
        out[(size_t)m * N + n0 + row] = from_float<TOut>(sv * uv);
      } else if constexpr (!RESID) {
        out[(size_t)m * N + n0 + row] = from_float<TOut>(s);
      }
    }
    if constexpr (RESID) {
      if (ksplit == 1) to_stream(m, row, s, true);
    }
  }
  if (ksplit == 1) return;
  // ---- the CTA of this row tile that arrives last adds the slices in order
  if (!cta_arrives_last(&g_skinny_arrivals[blockIdx.x], (unsigned int)ksplit, &is_last)) return;
  for (int idx = threadIdx.x; idx < RT * 16 * COLS; idx += WARPS * 32) {
    const int m = idx / (RT * 16), row = idx - m * (RT * 16);
    float s = 0.f, u = 0.f;
    if (m < M) {
      float sv[SK_MAX_SPLIT], uv[SK_MAX_SPLIT];
#pragma unroll
      for (int ks = 0; ks < SK_MAX_SPLIT; ++ks) {      // independent loads, summed in slice order
        const float* pp = g_skinny_partial + (size_t)ks * SK_SPLIT_MAX_ROWS * width + (size_t)m * width;
        sv[ks] = ks < ksplit ? __ldcg(pp + n0 + row) : 0.f;
        if constexpr (FUSE) uv[ks] = ks < ksplit ? __ldcg(pp + N + n0 + row) : 0.f;
      }
#pragma unroll
      for (int ks = 0; ks < SK_MAX_SPLIT; ++ks) {
        s += sv[ks];
        if constexpr (FUSE) u += uv[ks];
      }
      if constexpr (NORMX) {
        s *= rstd_s[m];
        u *= rstd_s[m];
      }
      if constexpr (FUSE) {
        const float gv = round_to<bf16>(s), uvv = round_to<bf16>(u);
        const float act = round_to<bf16>(gv / (1.f + expf(-gv)));
        out[(size_t)m * N + n0 + row] = from_float<TOut>(act * uvv);
      } else if constexpr (!RESID) {
        out[(size_t)m * N + n0 + row] = from_float<TOut>(s);
      }
    }
    if constexpr (RESID) to_stream(m, row, s, false);
  }
}

template <typename TOut, int NT, int RT, bool FUSE, int SK_PF, bool NORMX = false, bool RESID = false>
static int launch_skinny(const bf16* x, const bf16* w, TOut* out, int M, int N, int K, cudaStream_t stream,
                         const SkinnyNorm& nrm = SkinnyNorm()) {
  constexpr int TILES = FUSE ? 2 * RT : RT;
  const size_t smem = sizeof(float) * SK_WARPS * TILES * 16 * (8 * NT + 1);
  // Split K across CTAs when the row tiles alone leave most SMs idle.
  const int tiles = N / (16 * RT);
  int ksplit = 1;
  if (M <= SK_SPLIT_MAX_ROWS && (FUSE ? 2 * N : N) <= SK_SPLIT_MAX_COLS && tiles <= SK_MAX_TILES) {
    while (ksplit < SK_MAX_SPLIT && tiles * ksplit < 148 && K % (64 * ksplit) == 0 && K / (2 * ksplit) >= SK_KSTEP)
      ksplit *= 2;
  }
  constexpr bool CAN_RING = (!FUSE && RT == 1 && NT <= 2);
  const bool ring = CAN_RING && K / ksplit <= SK_PF * SK_KSTEP;
  // The tall form: when the row tiles alone leave SMs idle and a CTA of 16 warps can have its
  // whole share of the weights in flight (6 k blocks a warp: K up to 3,072), K is split between
  // the warps of one CTA only. Splitting it across CTAs instead costs a trip through global memory,
  // an arrival counter and a second pass by the last CTA, about 1.7 us at the end of a kernel in
  // which nothing else is left to overlap them (measured on B200 inside a decode step).
  if constexpr (CAN_RING && !NORMX) {
    if (ksplit > 1 && K <= SK_TALL_PF * SK_TALL_WARPS * 32) {
      auto tall = gemm_skinny_kernel<TOut, NT, RT, FUSE, SK_TALL_PF, true, NORMX, RESID, SK_TALL_WARPS>;
      const size_t tall_smem = sizeof(float) * SK_TALL_WARPS * TILES * 16 * (8 * NT + 1);
      return launch(tall, dim3(tiles, 1), SK_TALL_WARPS * 32, tall_smem, stream, x, w, out, M, N, K, nrm);
    }
  }
  void (*kern)(const bf16*, const bf16*, TOut*, int, int, int, SkinnyNorm) =
      gemm_skinny_kernel<TOut, NT, RT, FUSE, SK_PF, false, NORMX, RESID>;
  if constexpr (CAN_RING) {
    if (ring) kern = gemm_skinny_kernel<TOut, NT, RT, FUSE, SK_PF, true, NORMX, RESID>;
  }
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch(kern, dim3(tiles, ksplit), SK_THREADS, smem, stream, x, w, out, M, N, K, nrm);
}

// Weight row tiles per CTA: as many as still leave every SM a CTA (more tiles = each fragment of
// x is reused more often and less of L2's bandwidth goes to x).
static int row_tiles_for(int N, int most) {
  int rt = 1;
  while (rt * 2 <= most && N % (32 * rt) == 0 && N / (32 * rt) >= 148 * 4) rt *= 2;
  return rt;
}

// The streaming form, for matrices of very many rows (the output head: 151,936 x 1,024): a CTA
// takes row tiles blockIdx.x, + gridDim.x, ... one after the other, and asks for the weights of
// its next tile while the sums of the current one are still being added up and stored, so its
// requests never pause. (With one tile per CTA, a CTA's loads stop while it reduces and stores,
// and the next CTA on the SM starts with an empty pipeline: 16 rows on the head of 151,936 x 1,024
// take 184 us that way and 103 us in this form.)
// The rows of x are the same for every tile, so the CTA copies them to shared memory once and takes
// its B fragments from there: read from L2 for every tile instead, 16 rows of x were half as many
// bytes again as the weights themselves (134 us for that head inside a decode step of 16 rows, 73 us
// with 9 rows). A row of x in shared memory is K + 32 values long, so that the two rows that a
// quarter warp reads with one 16-byte load per lane fall into different halves of the banks.
// K must be a multiple of SK_ST_PF * 256, so that the ring of weight registers turns over in step
// with the tiles.
// A CTA takes its first tile by its index and claims every further one from a counter, one tile
// ahead: inside a decode step some CTAs start late (the kernels before and after hold part of the
// machine: the sampling kernel's CTAs are launched early and wait for this one), and with a fixed
// share of tiles per CTA the late ones set the kernel's time (16 rows on that head: 59 us alone,
// 105 us inside a step). The CTA that finishes last puts the counters back, so launches of this
// kernel must not overlap (as for the products that split K across CTAs).
constexpr int SK_ST_PF = 4;
constexpr int SK_ST_XPAD = 32;
static __device__ unsigned int g_stream_claimed, g_stream_finished;
template <typename TOut, int NT, int RT>
__global__ void __launch_bounds__(SK_THREADS, 2) gemm_skinny_stream_kernel(const bf16* __restrict__ x,
                                                                        const bf16* __restrict__ w,
                                                                        TOut* __restrict__ out, int M, int N, int K) {
  constexpr int PF = SK_ST_PF, COLS = 8 * NT, CS = COLS + 1;      // CS: see gemm_skinny_kernel
  extern __shared__ __align__(16) float red[];   // [SK_WARPS][RT][16][CS], then x [COLS][K + SK_ST_XPAD] bf16
  bf16* xs = reinterpret_cast<bf16*>(red + SK_WARPS * RT * 16 * CS);
  __shared__ int next_tile_s;
  const int xstride = K + SK_ST_XPAD;
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int tiles = N / (16 * RT);
  const size_t tile_stride = (size_t)16 * RT * K;
  const bf16* lane_w = w + (size_t)g * K + 8 * t + warp * 32;      // row g of tile 0, this lane's k offset
  uint4 ring[PF][RT][2];
  {
    const bf16* base = lane_w + (size_t)blockIdx.x * tile_stride;
#pragma unroll
    for (int p = 0; p < PF; ++p)
#pragma unroll
      for (int r = 0; r < RT; ++r) {
        ring[p][r][0] = ld_stream(base + (size_t)(r * 16) * K + p * SK_KSTEP);
        ring[p][r][1] = ld_stream(base + (size_t)(r * 16 + 8) * K + p * SK_KSTEP);
      }
  }
  pdl_wait();
  if (threadIdx.x == 0) next_tile_s = (int)(gridDim.x + atomicAdd(&g_stream_claimed, 1u));
  // x -> shared memory, rows from M on as zeros
  {
    const int per_row = K / 8;
    for (int idx = threadIdx.x; idx < COLS * per_row; idx += SK_THREADS) {
      const int m = idx / per_row, c = idx - m * per_row;
      const uint4 v = m < M ? ld_cg(x + (size_t)m * K + 8 * c) : make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(xs + (size_t)m * xstride + 8 * c) = v;
    }
  }
  __syncthreads();
  const bf16* xrow[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) xrow[j] = xs + (size_t)(8 * j + g) * xstride + 8 * t + warp * 32;
  int next_tile = next_tile_s;
  for (int tile = blockIdx.x; tile < tiles;) {
    const bool has_next = next_tile < tiles;
    const bf16* cur = lane_w + (size_t)tile * tile_stride;
    const bf16* nxt_tile = lane_w + (size_t)next_tile * tile_stride;
    // the tile after the next one: claimed now, needed when this tile is done
    int after = tiles;
    if (threadIdx.x == 0 && has_next) after = (int)(gridDim.x + atomicAdd(&g_stream_claimed, 1u));
    float acc[RT][NT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[r][j][e] = 0.f;
    for (int kb0 = 0; kb0 < K; kb0 += PF * SK_KSTEP) {
#pragma unroll
      for (int p = 0; p < PF; ++p) {
        const int kb = kb0 + p * SK_KSTEP;
        uint4 b[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) b[j] = *reinterpret_cast<const uint4*>(xrow[j] + kb);
#pragma unroll
        for (int r = 0; r < RT; ++r)
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            mma_bf16_16816(acc[r][j], ring[p][r][0].x, ring[p][r][1].x, ring[p][r][0].y, ring[p][r][1].y, b[j].x, b[j].y);
            mma_bf16_16816(acc[r][j], ring[p][r][0].z, ring[p][r][1].z, ring[p][r][0].w, ring[p][r][1].w, b[j].z, b[j].w);
          }
        // the registers are free again: the same k block of the next round, or of the next tile
        const int ahead = kb + PF * SK_KSTEP;
        if (ahead < K || has_next) {
          const bf16* src = ahead < K ? cur + ahead : nxt_tile + (ahead - K);
#pragma unroll
          for (int r = 0; r < RT; ++r) {
            ring[p][r][0] = ld_stream(src + (size_t)(r * 16) * K);
            ring[p][r][1] = ld_stream(src + (size_t)(r * 16 + 8) * K);
          }
        }
      }
    }
    float* mine = red + (size_t)warp * RT * 16 * CS;
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        float* tl = mine + (size_t)r * 16 * CS + j * 8;
        tl[g * CS + 2 * t] = acc[r][j][0];
        tl[g * CS + 2 * t + 1] = acc[r][j][1];
        tl[(g + 8) * CS + 2 * t] = acc[r][j][2];
        tl[(g + 8) * CS + 2 * t + 1] = acc[r][j][3];
      }
    __syncthreads();
    const int n0 = tile * 16 * RT;
    for (int idx = threadIdx.x; idx < RT * 16 * COLS; idx += SK_THREADS) {
      const int m = idx / (RT * 16), row = idx - m * (RT * 16);
      if (m < M) {
        float sum = 0.f;
#pragma unroll
        for (int wq = 0; wq < SK_WARPS; ++wq) sum += red[(size_t)wq * RT * 16 * CS + row * CS + m];   // a fixed order
        out[(size_t)m * N + n0 + row] = from_float<TOut>(sum);
      }
    }
    if (threadIdx.x == 0) next_tile_s = after;
    __syncthreads();      // the sums are read; the next tile may overwrite them
    tile = next_tile;
    next_tile = next_tile_s;
  }
  if (threadIdx.x == 0 && atomicAdd(&g_stream_finished, 1u) == gridDim.x - 1) {
    g_stream_claimed = 0;      // every CTA has made its last claim
    g_stream_finished = 0;
    __threadfence();
  }
}

// Shared memory of the streaming form: the partial sums and the rows of x.
template <int NT, int RT>
static size_t skinny_stream_smem(int K) {
  return sizeof(float) * SK_WARPS * RT * 16 * (8 * NT + 1) + sizeof(bf16) * 8 * NT * (size_t)(K + SK_ST_XPAD);
}
constexpr size_t SK_ST_MAX_SMEM = 200 * 1024;      // one CTA an SM; up to half of it, two

template <typename TOut, int NT, int RT>
static int launch_skinny_stream(const bf16* x, const bf16* w, TOut* out, int M, int N, int K, cudaStream_t stream) {
  const int tiles = N / (16 * RT);
  const size_t smem = skinny_stream_smem<NT, RT>(K);
  auto kern = gemm_skinny_stream_kernel<TOut, NT, RT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int ctas = (smem <= SK_ST_MAX_SMEM / 2 ? 2 : 1) * 148;
  return launch(kern, dim3(tiles < ctas ? tiles : ctas), SK_THREADS, smem, stream, x, w, out, M, N, K);
}

// The forms of up to 16 rows with 8 weight rows per tile instead of 16: the operands change places, x is
// the A operand (its rows g, and g + 8 where there are more than 8) and the weights the B operand (weight
// row g, 8 per tile), so a lane still loads 8 consecutive k of "its" weight row and of "its" x row
// for two m16n8k16. An SM takes in about 60 GB/s whatever the kernel, so a product lasts as long as
// the SM with the most weights needs, and units of half the size spread better: N = 1,024 (o, down) is
// 64 CTAs of 64 or 96 KB in the 16-row tall form and 128 CTAs of 32 or 48 KB here; the 192 CTAs of
// gate/up (two of 64 KB on 44 of the 148 SMs) become 384 of 32 KB (three on 88 SMs). Measured on B200,
// Qwen3-0.6B sizes, ms a decode step with o and down in this form: batch 1 0.758 -> 0.708, batch 8
// 0.841 -> 0.829; with gate/up too 0.683 and 0.816. K is split between the warps of the CTA and all its weights are in flight at once
// (K <= PF * WARPS * 32). FUSE, NORMX, RESID as in gemm_skinny_kernel; RESID leaves the sums of
// squares per 8 columns (N / 8 parts a row).
// XR = 1: up to 8 rows of x; XR = 2: up to 16 (the tile's rows g + 8 are then x rows too).
template <typename TOut, bool FUSE, bool NORMX, bool RESID, int WARPS, int PF, int XR>
__global__ void __launch_bounds__(WARPS * 32) gemm_skinny_h8_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                                   TOut* __restrict__ out, int M, int N, int K,
                                                                   SkinnyNorm nrm) {
  static_assert(!(RESID && FUSE) && WARPS >= 8 && (XR == 1 || XR == 2), "");
  constexpr int KSTEP = WARPS * 32, CS = 9, TILES = FUSE ? 2 : 1, ROWS = 8 * XR;
  __shared__ float red[WARPS * TILES * ROWS * CS];      // [warp][tile][x row][weight row], rows padded by one word
  __shared__ float rstd_s[ROWS];
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 8;
  const bf16* wrow[TILES];
#pragma unroll
  for (int r = 0; r < TILES; ++r) wrow[r] = w + (size_t)(r * N + n0 + g) * K + 8 * t + warp * 32;
  uint4 ring[PF][TILES];
#pragma unroll
  for (int p = 0; p < PF; ++p)
    if (warp * 32 + p * KSTEP < K) {
#pragma unroll
      for (int r = 0; r < TILES; ++r) ring[p][r] = ld_stream(wrow[r] + p * KSTEP);
    }
  pdl_wait();
  // this thread's output (x row, weight row): RESID fetches the stream's value now and uses it at the end
  const int om = threadIdx.x >> 3, orow = threadIdx.x & 7;
  float resid_before = 0.f;
  if constexpr (RESID) {
    if (threadIdx.x < 8 * ROWS && om < M) resid_before = ld_cg_f32(nrm.resid_out + (size_t)om * N + n0 + orow);
  }
  // NORMX: warp m adds up the parts of the sums of squares of rows m and m + 8 once the products are done
  float ssq[XR][4];
  if constexpr (NORMX) {
#pragma unroll
    for (int h = 0; h < XR; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = warp + 8 * h, p = lane + 32 * i;
        ssq[h][i] = (warp < 8 && m < M && p < nrm.parts) ? ld_cg_f32(nrm.sumsq + m * nrm.parts + p) : 0.f;
      }
  }
  const bf16* xbase = NORMX ? nrm.resid16 : x;
  uint4 xring[PF][XR], wring[NORMX ? PF : 1];
#pragma unroll
  for (int p = 0; p < PF; ++p) {
    const bool in = warp * 32 + p * KSTEP < K;
#pragma unroll
    for (int h = 0; h < XR; ++h) {
      const int m = g + 8 * h;
      xring[p][h] = (m < M && in) ? ld_cached(xbase + (size_t)m * K + 8 * t + warp * 32 + p * KSTEP) : make_uint4(0u, 0u, 0u, 0u);
    }
    if constexpr (NORMX) wring[p] = in ? ld_cached(nrm.weight + 8 * t + warp * 32 + p * KSTEP) : make_uint4(0u, 0u, 0u, 0u);
  }
  float acc[TILES][4];
#pragma unroll
  for (int r = 0; r < TILES; ++r)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[r][e] = 0.f;
#pragma unroll
  for (int p = 0; p < PF; ++p) {
    if (warp * 32 + p * KSTEP < K) {
      uint4 a = xring[p][0], a8 = make_uint4(0u, 0u, 0u, 0u);
      if constexpr (XR == 2) a8 = xring[p][1];
      if constexpr (NORMX) {
        a = normed_fragment(a, wring[p]);
        if constexpr (XR == 2) a8 = normed_fragment(a8, wring[p]);
      }
#pragma unroll
      for (int r = 0; r < TILES; ++r) {
        mma_bf16_16816(acc[r], a.x, a8.x, a.y, a8.y, ring[p][r].x, ring[p][r].y);
        mma_bf16_16816(acc[r], a.z, a8.z, a.w, a8.w, ring[p][r].z, ring[p][r].w);
      }
    }
  }
  if constexpr (NORMX) {
#pragma unroll
    for (int h = 0; h < XR; ++h) {
      const int m = warp + 8 * h;
      const float ss = warp_sum((ssq[h][0] + ssq[h][1]) + (ssq[h][2] + ssq[h][3]));      // a fixed order
      if (lane == 0 && warp < 8 && m < M) rstd_s[m] = rsqrtf(ss / (float)K + nrm.eps);
    }
  }
  // acc[r][0], [1]: x row g, weight rows 2 t and 2 t + 1 of tile r; acc[r][2], [3]: x row g + 8
#pragma unroll
  for (int r = 0; r < TILES; ++r)
#pragma unroll
    for (int h = 0; h < XR; ++h) {
      red[((warp * TILES + r) * ROWS + g + 8 * h) * CS + 2 * t] = acc[r][2 * h];
      red[((warp * TILES + r) * ROWS + g + 8 * h) * CS + 2 * t + 1] = acc[r][2 * h + 1];
    }
  __syncthreads();
  if (threadIdx.x >= 8 * ROWS) return;      // whole warps: ROWS x rows x 8 weight rows
  float ps[WARPS], pu[FUSE ? WARPS : 1], s = 0.f, u = 0.f;
#pragma unroll
  for (int wq = 0; wq < WARPS; ++wq) {
    ps[wq] = red[((wq * TILES) * ROWS + om) * CS + orow];
    if constexpr (FUSE) pu[wq] = red[((wq * TILES + 1) * ROWS + om) * CS + orow];
  }
#pragma unroll
  for (int wq = 0; wq < WARPS; ++wq) {      // a fixed order
    s += ps[wq];
    if constexpr (FUSE) u += pu[wq];
  }
  if constexpr (NORMX) {
    const float rstd = om < M ? rstd_s[om] : 0.f;
    s *= rstd;
    u *= rstd;
  }
  if constexpr (RESID) {
    float r = 0.f;
    if (om < M) {
      r = resid_before + round_to<bf16>(s);
      nrm.resid_out[(size_t)om * N + n0 + orow] = r;
      nrm.resid16_out[(size_t)om * N + n0 + orow] = from_float<bf16>(r);
    }
    float sq = r * r;
    sq += __shfl_xor_sync(0xffffffffu, sq, 4);
    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
    if (orow == 0 && om < M) nrm.sumsq_out[om * gridDim.x + blockIdx.x] = sq;
  } else if (om < M) {
    if constexpr (FUSE) {
      // rounding points of the unfused path: product -> bf16, silu -> bf16, times up -> bf16
      const float gv = round_to<bf16>(s), uv = round_to<bf16>(u);
      const float sv = round_to<bf16>(gv / (1.f + expf(-gv)));
      out[(size_t)om * N + n0 + orow] = from_float<TOut>(sv * uv);
    } else {
      out[(size_t)om * N + n0 + orow] = from_float<TOut>(s);
    }
  }
}

// Whether tiles of 8 weight rows spread an output of N columns better over the SMs than tiles of 16:
// the SM with the most tiles then holds fewer weight rows.
static bool h8_spreads_better(int N) {
  const int t8 = N / 8, t16 = N / 16;      // only where tiles of 16 take fewer than two rounds: very tall matrices stream
  return N % 8 == 0 && t16 < 2 * 148 && ((t8 + 147) / 148) * 8 < ((t16 + 147) / 148) * 16;
}
constexpr int SK_H8_TALL_WARPS = 16, SK_H8_TALL_PF = 6;      // o and down: K up to 3,072
constexpr int SK_H8_WARPS = 8, SK_H8_PF = 4;                 // the products that normalise the stream: K up to 1,024
// Whether ts_gemm_skinny_to_stream takes the 8-row form for this shape; it then leaves N / 8 parts of
// the sums of squares per row instead of N / 16 (the consumer adds up at most 128).
static bool to_stream_takes_h8(int M, int N, int K) {
  return M <= 16 && h8_spreads_better(N) && N / 8 <= 128 && K <= SK_H8_TALL_PF * SK_H8_TALL_WARPS * 32;
}
static bool normed_takes_h8(int M, int N, int K) { return M <= 16 && h8_spreads_better(N) && K <= SK_H8_PF * SK_H8_WARPS * 32; }
// The plain and the SwiGLU product of up to 16 rows: narrow outputs take the tall CTAs, wide ones CTAs of 8 warps.
template <typename TOut, bool FUSE>
static int launch_h8_plain(const bf16* x, const bf16* w, TOut* out, int M, int N, int K, cudaStream_t stream) {
  const SkinnyNorm nrm = SkinnyNorm();
  if (K <= SK_H8_PF * SK_H8_WARPS * 32) {
    if (M <= 8) return launch(gemm_skinny_h8_kernel<TOut, FUSE, false, false, SK_H8_WARPS, SK_H8_PF, 1>, N / 8, SK_H8_WARPS * 32, 0, stream, x, w, out, M, N, K, nrm);
    return launch(gemm_skinny_h8_kernel<TOut, FUSE, false, false, SK_H8_WARPS, SK_H8_PF, 2>, N / 8, SK_H8_WARPS * 32, 0, stream, x, w, out, M, N, K, nrm);
  }
  if (M <= 8) return launch(gemm_skinny_h8_kernel<TOut, FUSE, false, false, SK_H8_TALL_WARPS, SK_H8_TALL_PF, 1>, N / 8, SK_H8_TALL_WARPS * 32, 0, stream, x, w, out, M, N, K, nrm);
  return launch(gemm_skinny_h8_kernel<TOut, FUSE, false, false, SK_H8_TALL_WARPS, SK_H8_TALL_PF, 2>, N / 8, SK_H8_TALL_WARPS * 32, 0, stream, x, w, out, M, N, K, nrm);
}
static bool plain_takes_h8(int M, int N, int K) { return M <= 16 && h8_spreads_better(N) && K <= SK_H8_TALL_PF * SK_H8_TALL_WARPS * 32; }

template <typename TOut, int NT>
static int dispatch_skinny_nt(const bf16* x, const bf16* w, TOut* out, int M, int N, int K, cudaStream_t stream) {
  const int rt = row_tiles_for(N, 2);
  if constexpr (NT <= 2) {
    // up to 16 rows and at least eight tiles for each CTA (the head of 151,936 x 1,024 inside a decode
    // step: 8 rows 62 us with one tile per CTA and 53 us in this form; 16 rows 53 us)
    if (rt == 2 && K % (SK_ST_PF * SK_KSTEP) == 0 && N / 32 >= 8 * 2 * 148 && skinny_stream_smem<NT, 2>(K) <= SK_ST_MAX_SMEM)
      return launch_skinny_stream<TOut, NT, 2>(x, w, out, M, N, K, stream);
  }
  if (rt == 2) return launch_skinny<TOut, NT, 2, false, 4>(x, w, out, M, N, K, stream);
  return launch_skinny<TOut, NT, 1, false, 4>(x, w, out, M, N, K, stream);
}

template <typename TOut>
static int dispatch_skinny(const bf16* x, const bf16* w, TOut* out, int M, int N, int K, cudaStream_t stream) {
  if (plain_takes_h8(M, N, K)) return launch_h8_plain<TOut, false>(x, w, out, M, N, K, stream);
  if (M <= 8) return dispatch_skinny_nt<TOut, 1>(x, w, out, M, N, K, stream);
  if (M <= 16) return dispatch_skinny_nt<TOut, 2>(x, w, out, M, N, K, stream);
  if (M <= 32) return dispatch_skinny_nt<TOut, 4>(x, w, out, M, N, K, stream);
  return dispatch_skinny_nt<TOut, 8>(x, w, out, M, N, K, stream);
}

template <int NT>
static int dispatch_swiglu_nt(const bf16* x, const bf16* w, bf16* out, int M, int inter, int K, cudaStream_t stream) {
  return launch_skinny<bf16, NT, 1, true, 4>(x, w, out, M, inter, K, stream);
}

}  // namespace ts

using namespace ts;

extern "C" int ts_gemm_skinny_max_rows() { return 64; }

extern "C" int ts_gemm_skinny(const void* x, const void* w, void* out, int M, int N, int K, int out_dtype,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || K % 32 != 0 || N % 16 != 0) return TS_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return TS_ERR_UNSUPPORTED;
  if (out_dtype == TS_DTYPE_BF16)
    return dispatch_skinny<bf16>((const bf16*)x, (const bf16*)w, (bf16*)out, M, N, K, stream);
  if (out_dtype == TS_DTYPE_F32)
    return dispatch_skinny<float>((const bf16*)x, (const bf16*)w, (float*)out, M, N, K, stream);
  return TS_ERR_BAD_ARGUMENT;
}

// act[M, inter] = silu(x gate^T) * (x up^T) with w = [gate rows; up rows] of shape [2 inter, K].
extern "C" int ts_gemm_skinny_swiglu(const void* x, const void* w, void* out, int M, int inter, int K,
                                     cudaStream_t stream) {
  if (M <= 0 || inter <= 0) return 0;
  if (M > 32 || K <= 0 || K % 32 != 0 || inter % 16 != 0) return TS_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return TS_ERR_UNSUPPORTED;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)w;
  bf16* op = (bf16*)out;
  if (plain_takes_h8(M, inter, K)) return launch_h8_plain<bf16, true>(xp, wp, op, M, inter, K, stream);
  if (M <= 8) return dispatch_swiglu_nt<1>(xp, wp, op, M, inter, K, stream);
  if (M <= 16) return dispatch_swiglu_nt<2>(xp, wp, op, M, inter, K, stream);
  return dispatch_swiglu_nt<4>(xp, wp, op, M, inter, K, stream);
}

// out = rms_norm(resid) * w^T where the norm is made on the fly (NORMX above): resid16 [M, K] bf16,
// sumsq [M][parts] float (parts = K / 16 as the producer leaves them), norm_weight [K] bf16. M <= 16.
// swiglu != 0: w is [2 N, K] (gate rows, then up rows) and out = silu(gate) * up, [M, N] bf16.
extern "C" int ts_gemm_skinny_normed(const void* resid16, const float* sumsq, int parts, const void* norm_weight,
                                     float eps, const void* w, void* out, int M, int N, int K, int out_dtype,
                                     int swiglu, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || K % 32 != 0 || N % 16 != 0 || parts <= 0 || parts > 128) return TS_ERR_UNSUPPORTED;
  if (((uintptr_t)resid16 | (uintptr_t)w | (uintptr_t)norm_weight) & 15) return TS_ERR_UNSUPPORTED;
  SkinnyNorm nrm = SkinnyNorm();
  nrm.resid16 = (const bf16*)resid16; nrm.sumsq = sumsq; nrm.parts = parts; nrm.weight = (const bf16*)norm_weight; nrm.eps = eps;
  const bf16* wp = (const bf16*)w;
  if (normed_takes_h8(M, N, K) && out_dtype == TS_DTYPE_BF16) {
    const bf16* none = nullptr;
    if (swiglu && M <= 8)
      return launch(gemm_skinny_h8_kernel<bf16, true, true, false, SK_H8_WARPS, SK_H8_PF, 1>, N / 8, SK_H8_WARPS * 32, 0, stream, none, wp, (bf16*)out, M, N, K, nrm);
    if (swiglu)
      return launch(gemm_skinny_h8_kernel<bf16, true, true, false, SK_H8_WARPS, SK_H8_PF, 2>, N / 8, SK_H8_WARPS * 32, 0, stream, none, wp, (bf16*)out, M, N, K, nrm);
    if (M <= 8)
      return launch(gemm_skinny_h8_kernel<bf16, false, true, false, SK_H8_WARPS, SK_H8_PF, 1>, N / 8, SK_H8_WARPS * 32, 0, stream, none, wp, (bf16*)out, M, N, K, nrm);
    return launch(gemm_skinny_h8_kernel<bf16, false, true, false, SK_H8_WARPS, SK_H8_PF, 2>, N / 8, SK_H8_WARPS * 32, 0, stream, none, wp, (bf16*)out, M, N, K, nrm);
  }
  if (swiglu) {
    if (out_dtype != TS_DTYPE_BF16) return TS_ERR_BAD_ARGUMENT;
    if (M <= 8) return launch_skinny<bf16, 1, 1, true, 4, true, false>(nullptr, wp, (bf16*)out, M, N, K, stream, nrm);
    return launch_skinny<bf16, 2, 1, true, 4, true, false>(nullptr, wp, (bf16*)out, M, N, K, stream, nrm);
  }
  if (out_dtype == TS_DTYPE_BF16) {
    if (M <= 8) return launch_skinny<bf16, 1, 1, false, 4, true, false>(nullptr, wp, (bf16*)out, M, N, K, stream, nrm);
    return launch_skinny<bf16, 2, 1, false, 4, true, false>(nullptr, wp, (bf16*)out, M, N, K, stream, nrm);
  }
  if (out_dtype == TS_DTYPE_F32) {
    if (M <= 8) return launch_skinny<float, 1, 1, false, 4, true, false>(nullptr, wp, (float*)out, M, N, K, stream, nrm);
    return launch_skinny<float, 2, 1, false, 4, true, false>(nullptr, wp, (float*)out, M, N, K, stream, nrm);
  }
  return TS_ERR_BAD_ARGUMENT;
}

// resid[M, N] += bf16(x * w^T) in place, resid16 = bf16(resid), and sumsq_out[m * (N / 16) + n / 16]
// = sum over the 16 columns from n of the new resid[m, .]^2 (RESID above). M <= 16; sumsq_out
// holds M * N / 16 floats. Where ts_gemm_skinny_to_stream_parts(M, N, K) says so, the parts are of 8
// columns: sumsq_out[m * (N / 8) + n / 8], M * N / 8 floats (up to 2 N).
extern "C" int ts_gemm_skinny_to_stream_parts(int M, int N, int K) { return to_stream_takes_h8(M, N, K) ? N / 8 : N / 16; }

extern "C" int ts_gemm_skinny_to_stream(const void* x, const void* w, float* resid, void* resid16, float* sumsq_out,
                                        int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || K % 32 != 0 || N % 16 != 0) return TS_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return TS_ERR_UNSUPPORTED;
  SkinnyNorm nrm = SkinnyNorm();
  nrm.resid_out = resid; nrm.resid16_out = (bf16*)resid16; nrm.sumsq_out = sumsq_out;
  if (to_stream_takes_h8(M, N, K)) {
    if (M <= 8)
      return launch(gemm_skinny_h8_kernel<bf16, false, false, true, SK_H8_TALL_WARPS, SK_H8_TALL_PF, 1>, N / 8, SK_H8_TALL_WARPS * 32,
                    0, stream, (const bf16*)x, (const bf16*)w, (bf16*)nullptr, M, N, K, nrm);
    return launch(gemm_skinny_h8_kernel<bf16, false, false, true, SK_H8_TALL_WARPS, SK_H8_TALL_PF, 2>, N / 8, SK_H8_TALL_WARPS * 32,
                  0, stream, (const bf16*)x, (const bf16*)w, (bf16*)nullptr, M, N, K, nrm);
  }
  if (M <= 8)
    return launch_skinny<bf16, 1, 1, false, 4, false, true>((const bf16*)x, (const bf16*)w, (bf16*)nullptr, M, N, K, stream, nrm);
  return launch_skinny<bf16, 2, 1, false, 4, false, true>((const bf16*)x, (const bf16*)w, (bf16*)nullptr, M, N, K, stream, nrm);
}
