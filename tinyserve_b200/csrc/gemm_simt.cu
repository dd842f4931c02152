// out[M, N] = x[M, K] * w[N, K]^T on CUDA cores with 32-bit accumulation (no tensor cores,
// no reduced-precision mode): the matrix product of the true 32-bit path, and the fallback
// of the bf16 path for shapes the tensor-core kernels refuse. Any M, N, K.
//
// 64 x 64 output tile per CTA, K in steps of 16, 256 threads with a 4 x 4 register tile each.
// The sum over K runs in index order for every output, whatever M is, so a row's result does
// not depend on which other rows share the batch.
#define TS_PDL_CLASS PDL_OTHER
#include "common.cuh"

namespace ts {

constexpr int GM = 64, GN = 64, GK = 16, GTHREADS = 256;

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(GTHREADS) gemm_simt_kernel(const TIn* __restrict__ x, const TIn* __restrict__ w,
                                                             TOut* __restrict__ out, int M, int N, int K) {
  __shared__ float As[GK][GM + 4];
  __shared__ float Bs[GK][GN + 4];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * GM, n0 = blockIdx.x * GN;
  const int ty = tid >> 4, tx = tid & 15;
  // loading: thread -> row (tid / 4), 4 consecutive k starting at (tid % 4) * 4
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += GK) {
    float av[4], bv[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int am = m0 + lrow, bn = n0 + lrow;
      av[e] = (am < M && k < K) ? to_float(x[(size_t)am * K + k]) : 0.f;
      bv[e] = (bn < N && k < K) ? to_float(w[(size_t)bn * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      As[lk + e][lrow] = av[e];
      Bs[lk + e][lrow] = bv[e];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(size_t)m * N + n] = from_float<TOut>(acc[i][j]);
    }
  }
}

}  // namespace ts

using namespace ts;

// in_dtype: type of x and w; out_dtype: type of out (float output from bf16 inputs is allowed).
extern "C" int ts_gemm_simt(const void* x, const void* w, void* out, int M, int N, int K, int in_dtype,
                            int out_dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return TS_ERR_BAD_ARGUMENT;
  dim3 grid((N + GN - 1) / GN, (M + GM - 1) / GM);
  if (in_dtype == TS_DTYPE_F32 && out_dtype == TS_DTYPE_F32)
    return launch(gemm_simt_kernel<float, float>, grid, GTHREADS, 0, stream, (const float*)x, (const float*)w, (float*)out, M, N, K);
  if (in_dtype == TS_DTYPE_BF16 && out_dtype == TS_DTYPE_BF16)
    return launch(gemm_simt_kernel<bf16, bf16>, grid, GTHREADS, 0, stream, (const bf16*)x, (const bf16*)w, (bf16*)out, M, N, K);
  if (in_dtype == TS_DTYPE_BF16 && out_dtype == TS_DTYPE_F32)
    return launch(gemm_simt_kernel<bf16, float>, grid, GTHREADS, 0, stream, (const bf16*)x, (const bf16*)w, (float*)out, M, N, K);
  return TS_ERR_BAD_ARGUMENT;
}
