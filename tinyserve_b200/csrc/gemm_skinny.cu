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
// Needs K % 32 == 0 and N % 16 == 0 (the launcher reports TS_ERR_UNSUPPORTED otherwise and the
// caller takes another kernel).
#define TS_PDL_CLASS PDL_SKINNY
#include "common.cuh"

namespace ts {

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_KSTEP = SK_WARPS * 32;    // distance between a warp's k blocks
constexpr int SK_MAX_SPLIT = 8;
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
template <typename TOut, int NT, int RT, bool FUSE, int SK_PF, bool XRING>
__global__ void __launch_bounds__(SK_THREADS) gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                                 TOut* __restrict__ out, int M, int N, int K) {
  constexpr int TILES = FUSE ? 2 * RT : RT;
  constexpr int COLS = 8 * NT;
  extern __shared__ float red[];   // [SK_WARPS][TILES][16][COLS]
  __shared__ int is_last;
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
    const int kb = k_lo + warp * 32 + p * SK_KSTEP;
    if (kb < k_hi) {
#pragma unroll
      for (int r = 0; r < TILES; ++r) {
        ring[p][r][0] = ld_stream(wrow[r][0] + kb);
        ring[p][r][1] = ld_stream(wrow[r][1] + kb);
      }
    }
  }
  pdl_wait();

  float acc[TILES][NT][4];
#pragma unroll
  for (int r = 0; r < TILES; ++r)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[r][j][e] = 0.f;
  const bf16* xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int m = 8 * j + g;
    xok[j] = m < M;
    xrow[j] = x + (size_t)(xok[j] ? m : 0) * K + 8 * t;
  }
  // XRING: the fragments of x are fetched as far ahead as the weights. Chosen when a warp has so
  // few k blocks that all its loads go out at once and nothing later waits for L2; with long
  // loops the extra registers would cost more in occupancy than the prefetch gains.
  uint4 xring[XRING ? SK_PF : 1][NT];
  if constexpr (XRING) {
#pragma unroll
    for (int p = 0; p < SK_PF; ++p) {
      const int kb = k_lo + warp * 32 + p * SK_KSTEP;
#pragma unroll
      for (int j = 0; j < NT; ++j)
        xring[p][j] = (kb < k_hi && xok[j]) ? ld_cached(xrow[j] + kb) : make_uint4(0u, 0u, 0u, 0u);
    }
  }

  for (int kb0 = k_lo + warp * 32; kb0 < k_hi; kb0 += SK_PF * SK_KSTEP) {
#pragma unroll
    for (int p = 0; p < SK_PF; ++p) {
      const int kb = kb0 + p * SK_KSTEP;
      if (kb < k_hi) {
        uint4 a[TILES][2];
#pragma unroll
        for (int r = 0; r < TILES; ++r) { a[r][0] = ring[p][r][0]; a[r][1] = ring[p][r][1]; }
        uint4 b[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          if constexpr (XRING) b[j] = xring[p][j];
          else b[j] = xok[j] ? ld_cached(xrow[j] + kb) : make_uint4(0u, 0u, 0u, 0u);
        }
        const int nxt = kb + SK_PF * SK_KSTEP;
        if (nxt < k_hi) {
#pragma unroll
          for (int r = 0; r < TILES; ++r) {
            ring[p][r][0] = ld_stream(wrow[r][0] + nxt);
            ring[p][r][1] = ld_stream(wrow[r][1] + nxt);
          }
          if constexpr (XRING) {
#pragma unroll
            for (int j = 0; j < NT; ++j) xring[p][j] = xok[j] ? ld_cached(xrow[j] + nxt) : make_uint4(0u, 0u, 0u, 0u);
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

  // partial sums of this warp -> shared memory; element (row, col) of tile (r, j)
  float* mine = red + (size_t)warp * TILES * 16 * COLS;
#pragma unroll
  for (int r = 0; r < TILES; ++r)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      float* tile = mine + (size_t)r * 16 * COLS + j * 8;
      tile[g * COLS + 2 * t] = acc[r][j][0];
      tile[g * COLS + 2 * t + 1] = acc[r][j][1];
      tile[(g + 8) * COLS + 2 * t] = acc[r][j][2];
      tile[(g + 8) * COLS + 2 * t + 1] = acc[r][j][3];
    }
  __syncthreads();
  // thread -> (column m, weight row): consecutive threads take consecutive weight rows, so a
  // column of the result is written as one run of out[m, n0 .. n0 + 16 RT).
  const int width = FUSE ? 2 * N : N;                 // columns of a partial row
  float* part = g_skinny_partial + (size_t)blockIdx.y * SK_SPLIT_MAX_ROWS * width;
  for (int idx = threadIdx.x; idx < RT * 16 * COLS; idx += SK_THREADS) {
    const int m = idx / (RT * 16), row = idx - m * (RT * 16);
    if (m < M) {
      float s = 0.f, u = 0.f;
#pragma unroll
      for (int wq = 0; wq < SK_WARPS; ++wq) s += red[(size_t)wq * TILES * 16 * COLS + row * COLS + m];
      if constexpr (FUSE) {
#pragma unroll
        for (int wq = 0; wq < SK_WARPS; ++wq) u += red[(size_t)wq * TILES * 16 * COLS + (RT * 16 + row) * COLS + m];
      }
      if (ksplit > 1) {
        part[(size_t)m * width + n0 + row] = s;
        if constexpr (FUSE) part[(size_t)m * width + N + n0 + row] = u;
      } else if constexpr (FUSE) {
        // rounding points of the unfused path: product -> bf16, silu -> bf16, times up -> bf16
        const float gv = round_to<bf16>(s), uv = round_to<bf16>(u);
        const float sv = round_to<bf16>(gv / (1.f + expf(-gv)));
        out[(size_t)m * N + n0 + row] = from_float<TOut>(sv * uv);
      } else {
        out[(size_t)m * N + n0 + row] = from_float<TOut>(s);
      }
    }
  }
  if (ksplit == 1) return;
  // ---- the CTA of this row tile that arrives last adds the slices in order
  if (!cta_arrives_last(&g_skinny_arrivals[blockIdx.x], (unsigned int)ksplit, &is_last)) return;
  for (int idx = threadIdx.x; idx < RT * 16 * COLS; idx += SK_THREADS) {
    const int m = idx / (RT * 16), row = idx - m * (RT * 16);
    if (m < M) {
      float sv[SK_MAX_SPLIT], uv[SK_MAX_SPLIT];
#pragma unroll
      for (int ks = 0; ks < SK_MAX_SPLIT; ++ks) {      // independent loads, summed in slice order
        const float* pp = g_skinny_partial + (size_t)ks * SK_SPLIT_MAX_ROWS * width + (size_t)m * width;
        sv[ks] = ks < ksplit ? __ldcg(pp + n0 + row) : 0.f;
        if constexpr (FUSE) uv[ks] = ks < ksplit ? __ldcg(pp + N + n0 + row) : 0.f;
      }
      float s = 0.f, u = 0.f;
#pragma unroll
      for (int ks = 0; ks < SK_MAX_SPLIT; ++ks) {
        s += sv[ks];
        if constexpr (FUSE) u += uv[ks];
      }
      if constexpr (FUSE) {
        const float gv = round_to<bf16>(s), uvv = round_to<bf16>(u);
        const float act = round_to<bf16>(gv / (1.f + expf(-gv)));
        out[(size_t)m * N + n0 + row] = from_float<TOut>(act * uvv);
      } else {
        out[(size_t)m * N + n0 + row] = from_float<TOut>(s);
      }
    }
  }
}

template <typename TOut, int NT, int RT, bool FUSE, int SK_PF>
static int launch_skinny(const bf16* x, const bf16* w, TOut* out, int M, int N, int K, cudaStream_t stream) {
  constexpr int TILES = FUSE ? 2 * RT : RT;
  const size_t smem = sizeof(float) * SK_WARPS * TILES * 16 * 8 * NT;
  // Split K across CTAs when the row tiles alone leave most SMs idle.
  const int tiles = N / (16 * RT);
  int ksplit = 1;
  if (M <= SK_SPLIT_MAX_ROWS && (FUSE ? 2 * N : N) <= SK_SPLIT_MAX_COLS && tiles <= SK_MAX_TILES) {
    while (ksplit < SK_MAX_SPLIT && tiles * ksplit < 148 && K % (64 * ksplit) == 0 && K / (2 * ksplit) >= SK_KSTEP)
      ksplit *= 2;
  }
  constexpr bool CAN_RING = (!FUSE && RT == 1 && NT == 1);
  const bool ring = CAN_RING && K / ksplit <= SK_PF * SK_KSTEP;
  void (*kern)(const bf16*, const bf16*, TOut*, int, int, int) = gemm_skinny_kernel<TOut, NT, RT, FUSE, SK_PF, false>;
  if constexpr (CAN_RING) {
    if (ring) kern = gemm_skinny_kernel<TOut, NT, RT, FUSE, SK_PF, true>;
  }
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch(kern, dim3(tiles, ksplit), SK_THREADS, smem, stream, x, w, out, M, N, K);
}

// Weight row tiles per CTA: as many as still leave every SM a CTA (more tiles = each fragment of
// x is reused more often and less of L2's bandwidth goes to x).
static int row_tiles_for(int N, int most) {
  int rt = 1;
  while (rt * 2 <= most && N % (32 * rt) == 0 && N / (32 * rt) >= 148 * 4) rt *= 2;
  return rt;
}

template <typename TOut, int NT>
static int dispatch_skinny_nt(const bf16* x, const bf16* w, TOut* out, int M, int N, int K, cudaStream_t stream) {
  const int rt = row_tiles_for(N, 2);
  if (rt == 2) return launch_skinny<TOut, NT, 2, false, 4>(x, w, out, M, N, K, stream);
  return launch_skinny<TOut, NT, 1, false, 4>(x, w, out, M, N, K, stream);
}

template <typename TOut>
static int dispatch_skinny(const bf16* x, const bf16* w, TOut* out, int M, int N, int K, cudaStream_t stream) {
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
  if (M <= 8) return dispatch_swiglu_nt<1>(xp, wp, op, M, inter, K, stream);
  if (M <= 16) return dispatch_swiglu_nt<2>(xp, wp, op, M, inter, K, stream);
  return dispatch_swiglu_nt<4>(xp, wp, op, M, inter, K, stream);
}
