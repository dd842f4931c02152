// out[M, N] = x[M, K] * w[N, K]^T for a handful of rows (decode: M = live requests), bf16 in,
// 32-bit accumulation on the tensor cores, bf16 or float out.
//
// The product is memory-bound: every weight is read once and used M times. So the weights are
// the A operand (16 weight rows per mma tile), streamed straight from global memory into the
// mma fragments with 16-byte loads that never pass through shared memory, and the few rows of x
// are the B operand (8 columns per tile), read through L1. Each lane loads 8 consecutive k of
// "its" weight row and of "its" x row; which k feeds which slot of the mma does not matter as
// long as A and B agree, so those 8 values serve two m16n8k16 instructions without any shuffle.
// A CTA owns 16 * ROW_TILES weight rows; its 8 warps split K between them and add their partial
// sums in shared memory in a fixed order, so the result is deterministic.
//
// Needs K % 32 == 0 and N % 16 == 0 (the launcher reports TS_ERR_UNSUPPORTED otherwise and the
// caller takes another kernel).
#include "common.cuh"

namespace ts {

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cached(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
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

// NT = column tiles of 8 rows of x (M <= 8 * NT); RT = weight row tiles of 16 per CTA.
template <typename TOut, int NT, int RT>
__global__ void __launch_bounds__(SK_THREADS) gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                                 TOut* __restrict__ out, int M, int N, int K) {
  extern __shared__ float red[];   // [SK_WARPS][RT][16][8 * NT]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * (16 * RT);

  float acc[RT][NT][4];
#pragma unroll
  for (int r = 0; r < RT; ++r)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[r][j][e] = 0.f;

  const bf16* wrow[RT][2];
#pragma unroll
  for (int r = 0; r < RT; ++r) {
    wrow[r][0] = w + (size_t)(n0 + r * 16 + g) * K + 8 * t;
    wrow[r][1] = w + (size_t)(n0 + r * 16 + g + 8) * K + 8 * t;
  }
  const bf16* xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int m = 8 * j + g;
    xok[j] = m < M;
    xrow[j] = x + (size_t)(xok[j] ? m : 0) * K + 8 * t;
  }

  // warp `warp` takes k blocks warp, warp + 8, ... of 32
#pragma unroll 2
  for (int kb = warp * 32; kb < K; kb += SK_WARPS * 32) {
    uint4 a[RT][2];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
      a[r][0] = ld_stream(wrow[r][0] + kb);
      a[r][1] = ld_stream(wrow[r][1] + kb);
    }
    uint4 b[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) b[j] = xok[j] ? ld_cached(xrow[j] + kb) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        mma_bf16_16816(acc[r][j], a[r][0].x, a[r][1].x, a[r][0].y, a[r][1].y, b[j].x, b[j].y);
        mma_bf16_16816(acc[r][j], a[r][0].z, a[r][1].z, a[r][0].w, a[r][1].w, b[j].z, b[j].w);
      }
  }

  // partial sums of this warp -> shared memory; element (row, col) of tile (r, j)
  constexpr int COLS = 8 * NT;
  float* mine = red + (size_t)warp * RT * 16 * COLS;
#pragma unroll
  for (int r = 0; r < RT; ++r)
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
  for (int idx = threadIdx.x; idx < RT * 16 * COLS; idx += SK_THREADS) {
    const int m = idx / (RT * 16), row = idx - m * (RT * 16);
    if (m < M) {
      float s = 0.f;
#pragma unroll
      for (int wq = 0; wq < SK_WARPS; ++wq) s += red[(size_t)wq * RT * 16 * COLS + row * COLS + m];
      out[(size_t)m * N + n0 + row] = from_float<TOut>(s);
    }
  }
}

template <typename TOut, int NT, int RT>
static int launch_skinny(const bf16* x, const bf16* w, TOut* out, int M, int N, int K, cudaStream_t stream) {
  const size_t smem = sizeof(float) * SK_WARPS * RT * 16 * 8 * NT;
  auto kern = gemm_skinny_kernel<TOut, NT, RT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  kern<<<N / (16 * RT), SK_THREADS, smem, stream>>>(x, w, out, M, N, K);
  return launch_status();
}

template <typename TOut>
static int dispatch_skinny(const bf16* x, const bf16* w, TOut* out, int M, int N, int K, cudaStream_t stream) {
  // Two row tiles per CTA when that still leaves enough CTAs to fill the machine.
  const bool two = (N % 32 == 0) && (N / 32 >= 148 * 4);
#define TS_SKINNY(NT_)                                                                        \
  return two ? launch_skinny<TOut, NT_, 2>(x, w, out, M, N, K, stream)                        \
             : launch_skinny<TOut, NT_, 1>(x, w, out, M, N, K, stream)
  if (M <= 8) { TS_SKINNY(1); }
  if (M <= 16) { TS_SKINNY(2); }
  if (M <= 32) { TS_SKINNY(4); }
  TS_SKINNY(8);
#undef TS_SKINNY
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
