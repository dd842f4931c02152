// Embedding gather, residual-add + RMSNorm, rotary tables, SiLU-multiply.
//
// Rounding points follow the upstream engine's contract (src/tinyserve/layers.py:35-38,
// src/tinyserve/model.py:178-179): the norm is computed in 32-bit, cast to the model dtype,
// then multiplied by the weight in the model dtype; silu(gate) is rounded before the product.
// The residual stream itself is kept in 32-bit, so the residual sum is a 32-bit sum.
#define TS_PDL_CLASS PDL_ELEMENTWISE
#include "common.cuh"

namespace ts {

int g_programmatic_launch = 0;

// ---------------------------------------------------------------- embedding
// out[t, :] = float(table[tokens[t], :]).  A token id outside [0, vocab) yields a NaN row
// instead of an out-of-bounds read (the host checks ids too).
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                             float* __restrict__ out, int hidden, int vocab) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = tokens[t];
  float* o = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = __int_as_float(0x7fc00000);
    return;
  }
  const T* row = table + (size_t)id * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]);
}

// ------------------------------------------------------- residual add + RMSNorm
// x = resid[row] (+ delta[row]);  if rows == nullptr the sum is written back to resid.
// out[r] = T(x * rsqrt(mean(x^2) + eps)) * weight, the product rounded to T.
// The row is kept in shared memory between the two passes when it fits (cache_row).
template <typename T>
__global__ void add_rms_norm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                    const T* __restrict__ weight, T* __restrict__ out,
                                    const int* __restrict__ rows, int hidden, float eps, int cache_row) {
  extern __shared__ float xs[];
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* x = resid + (size_t)row * hidden;
  const T* d = delta ? delta + (size_t)row * hidden : nullptr;
  const bool write_back = (rows == nullptr) && (d != nullptr);
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = x[i];
    if (d) v += to_float(d[i]);
    if (write_back) x[i] = v;
    if (cache_row) xs[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v;
    if (cache_row) {
      v = xs[i];
    } else {
      v = x[i];
      if (d && !write_back) v += to_float(d[i]);
    }
    const float n = round_to<T>(v * rstd);
    o[i] = from_float<T>(n * to_float(weight[i]));
  }
}

// The same with 16-byte accesses on the 32-bit stream and 8-byte (bf16) or 16-byte (float)
// accesses on the rest: 4 elements per thread and step. Needs hidden % 4 == 0 and the row cache.
template <typename T>
__global__ void add_rms_norm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                        const T* __restrict__ weight, T* __restrict__ out,
                                        const int* __restrict__ rows, int hidden, float eps) {
  extern __shared__ float xs[];
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* x = resid + (size_t)row * hidden;
  const T* d = delta ? delta + (size_t)row * hidden : nullptr;
  const bool write_back = (rows == nullptr) && (d != nullptr);
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(x + i);
    if (d) {
      if constexpr (sizeof(T) == 2) {
        const uint2 raw = *reinterpret_cast<const uint2*>(d + i);
        v.x += __uint_as_float(raw.x << 16); v.y += __uint_as_float(raw.x & 0xffff0000u);
        v.z += __uint_as_float(raw.y << 16); v.w += __uint_as_float(raw.y & 0xffff0000u);
      } else {
        const float4 dv = *reinterpret_cast<const float4*>(d + i);
        v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
      }
    }
    if (write_back) *reinterpret_cast<float4*>(x + i) = v;
    *reinterpret_cast<float4*>(xs + i) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)r * hidden;
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xs + i);
    const float f[4] = {v.x, v.y, v.z, v.w};
    float w[4], res[4];
    if constexpr (sizeof(T) == 2) {
      const uint2 raw = *reinterpret_cast<const uint2*>(weight + i);
      w[0] = __uint_as_float(raw.x << 16); w[1] = __uint_as_float(raw.x & 0xffff0000u);
      w[2] = __uint_as_float(raw.y << 16); w[3] = __uint_as_float(raw.y & 0xffff0000u);
    } else {
      const float4 wv = *reinterpret_cast<const float4*>(weight + i);
      w[0] = wv.x; w[1] = wv.y; w[2] = wv.z; w[3] = wv.w;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) res[e] = round_to<T>(f[e] * rstd) * w[e];
    if constexpr (sizeof(T) == 2) {
      __nv_bfloat162 a = __floats2bfloat162_rn(res[0], res[1]), b = __floats2bfloat162_rn(res[2], res[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&a);
      pk.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(o + i) = pk;
    } else {
      *reinterpret_cast<float4*>(o + i) = make_float4(res[0], res[1], res[2], res[3]);
    }
  }
}

// ------------------------------------------------------------ rotary tables
// angle = position * inv_freq in float64; cos and sin in float64, rounded to float32.
__global__ void rope_tables_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                   float* __restrict__ cos_out, float* __restrict__ sin_out,
                                   int num_tokens, int half) {
  pdl_trigger();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= num_tokens * half) return;
  const int t = idx / half, i = idx - t * half;
  const double a = (double)positions[t] * inv_freq[i];
  double s, c;
  sincos(a, &s, &c);
  cos_out[idx] = (float)c;
  sin_out[idx] = (float)s;
}

// ------------------------------------------------------------- SiLU-multiply
// out[t, j] = T(silu(gate_up[t, j])) * gate_up[t, inter + j]
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
  pdl_trigger();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const size_t t = idx / inter;
    const int j = (int)(idx - t * inter);
    const float g = to_float(gate_up[t * 2 * inter + j]);
    const float u = to_float(gate_up[t * 2 * inter + inter + j]);
    const float s = round_to<T>(g / (1.f + expf(-g)));
    out[idx] = from_float<T>(s * u);
  }
}

// The same with 16-byte accesses; needs inter to be a multiple of the vector length.
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total_vecs) {
  constexpr int VEC = Vec<T>::N;
  pdl_trigger();
  pdl_wait();
  const int vecs_per_row = inter / VEC;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total_vecs; idx += stride) {
    const size_t t = idx / vecs_per_row;
    const int j = (int)(idx - t * vecs_per_row) * VEC;
    Vec<T> gv, uv, ov;
    gv.load(gate_up + t * 2 * inter + j);
    uv.load(gate_up + t * 2 * inter + inter + j);
    float g[VEC], u[VEC], o[VEC];
    gv.unpack(g);
    uv.unpack(u);
#pragma unroll
    for (int e = 0; e < VEC; ++e) o[e] = round_to<T>(g[e] / (1.f + expf(-g[e]))) * u[e];
    ov.pack(o);
    ov.store(out + t * inter + j);
  }
}

}  // namespace ts

using namespace ts;

// Turn programmatic dependent launch of this library's kernels on (1) or off (0).
// `mask` selects the kernel classes (1 elementwise, 2 skinny product, 4 attention, 8 tcgen05
// product, 16 sampling, 32 others); 0 turns it off, -1 turns it on for all.
extern "C" void ts_set_programmatic_launch(int mask) { g_programmatic_launch = mask; }
extern "C" int ts_get_programmatic_launch() { return g_programmatic_launch; }

// ---- kernel timeline (only in a library built with -DTS_TIMELINE; else always empty)
static void* g_tl_records[64];
static void* g_tl_counts[64];
static int g_tl_files = 0, g_tl_cap = 0;
extern "C" void ts_timeline_register(void* records, void* count, int cap) {
  if (g_tl_files < 64) {
    g_tl_records[g_tl_files] = records;
    g_tl_counts[g_tl_files] = count;
    ++g_tl_files;
    g_tl_cap = cap;
  }
}
// Copies up to `cap` records {kernel class and launch shape, start ns, wait-returned ns} of all
// source files to `out` (host memory, 3 words a record, unsorted) and empties the device side.
// Synchronises the device. Returns the number of records, or -1 on a CUDA error.
extern "C" int ts_timeline_read(unsigned long long* out, int cap) {
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  int n = 0;
  for (int f = 0; f < g_tl_files; ++f) {
    unsigned int count = 0;
    if (cudaMemcpy(&count, g_tl_counts[f], sizeof(count), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    int take = (int)(count < (unsigned int)g_tl_cap ? count : (unsigned int)g_tl_cap);
    if (take > cap - n) take = cap - n;
    if (take > 0 && cudaMemcpy(out + 3 * (size_t)n, g_tl_records[f], sizeof(unsigned long long) * 3 * take,
                               cudaMemcpyDeviceToHost) != cudaSuccess)
      return -1;
    n += take;
    if (cudaMemset(g_tl_counts[f], 0, sizeof(unsigned int)) != cudaSuccess) return -1;
  }
  return n;
}

extern "C" int ts_embed(const int* tokens, const void* table, float* out, int num_tokens, int hidden,
                        int vocab, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == TS_DTYPE_F32)
    return launch(embed_kernel<float>, num_tokens, threads, 0, stream, tokens, (const float*)table, out, hidden, vocab);
  if (dtype == TS_DTYPE_BF16)
    return launch(embed_kernel<bf16>, num_tokens, threads, 0, stream, tokens, (const bf16*)table, out, hidden, vocab);
  return TS_ERR_BAD_ARGUMENT;
}

// The same with a warp per row, for steps of many rows (prompts) and rows of 128 * NV values: every lane
// keeps its 4 NV values in registers between the two passes, all loads of a row are in flight at once,
// and the sum of squares is a warp reduction, with no shared memory and no block barrier. (A CTA per
// row at 1,024 columns is one 16-byte load per thread, two barriers and a store: 2,048 rows took
// 10.5 us on B200 for 24 MB that mostly lie in L2.)
template <typename T, int NV>
__global__ void __launch_bounds__(128) add_rms_norm_warp_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                                                const T* __restrict__ weight, T* __restrict__ out,
                                                                const int* __restrict__ rows, int num_rows, float eps) {
  constexpr int hidden = 128 * NV;
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= num_rows) return;
  const int row = rows ? rows[r] : r;
  float* x = resid + (size_t)row * hidden;
  const T* d = delta ? delta + (size_t)row * hidden : nullptr;
  const bool write_back = (rows == nullptr) && (d != nullptr);
  float4 v[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) v[j] = *reinterpret_cast<const float4*>(x + 4 * (lane + 32 * j));
  if (d) {
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = 4 * (lane + 32 * j);
      if constexpr (sizeof(T) == 2) {
        const uint2 raw = *reinterpret_cast<const uint2*>(d + i);
        v[j].x += __uint_as_float(raw.x << 16); v[j].y += __uint_as_float(raw.x & 0xffff0000u);
        v[j].z += __uint_as_float(raw.y << 16); v[j].w += __uint_as_float(raw.y & 0xffff0000u);
      } else {
        const float4 dv = *reinterpret_cast<const float4*>(d + i);
        v[j].x += dv.x; v[j].y += dv.y; v[j].z += dv.z; v[j].w += dv.w;
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    if (write_back) *reinterpret_cast<float4*>(x + 4 * (lane + 32 * j)) = v[j];
    ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)r * hidden;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = 4 * (lane + 32 * j);
    const float f[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
    float w[4], res[4];
    if constexpr (sizeof(T) == 2) {
      const uint2 raw = *reinterpret_cast<const uint2*>(weight + i);
      w[0] = __uint_as_float(raw.x << 16); w[1] = __uint_as_float(raw.x & 0xffff0000u);
      w[2] = __uint_as_float(raw.y << 16); w[3] = __uint_as_float(raw.y & 0xffff0000u);
    } else {
      const float4 wv = *reinterpret_cast<const float4*>(weight + i);
      w[0] = wv.x; w[1] = wv.y; w[2] = wv.z; w[3] = wv.w;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) res[e] = round_to<T>(f[e] * rstd) * w[e];
    if constexpr (sizeof(T) == 2) {
      __nv_bfloat162 a = __floats2bfloat162_rn(res[0], res[1]), b = __floats2bfloat162_rn(res[2], res[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&a);
      pk.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(o + i) = pk;
    } else {
      *reinterpret_cast<float4*>(o + i) = make_float4(res[0], res[1], res[2], res[3]);
    }
  }
}

template <typename T>
static int launch_add_rms_norm_warp(float* resid, const T* delta, const T* weight, T* out, const int* rows, int num_rows,
                                    int hidden, float eps, cudaStream_t stream) {
  const int grid = (num_rows + 3) / 4;
  switch (hidden / 128) {
    case 2: return launch(add_rms_norm_warp_kernel<T, 2>, grid, 128, 0, stream, resid, delta, weight, out, rows, num_rows, eps);
    case 4: return launch(add_rms_norm_warp_kernel<T, 4>, grid, 128, 0, stream, resid, delta, weight, out, rows, num_rows, eps);
    case 8: return launch(add_rms_norm_warp_kernel<T, 8>, grid, 128, 0, stream, resid, delta, weight, out, rows, num_rows, eps);
    default: return launch(add_rms_norm_warp_kernel<T, 16>, grid, 128, 0, stream, resid, delta, weight, out, rows, num_rows, eps);
  }
}
constexpr int NORM_WARP_ROWS = 256;      // from this many rows on a warp takes a row

extern "C" int ts_add_rms_norm(float* resid, const void* delta, const void* weight, void* out,
                               const int* rows, int num_rows, int hidden, float eps, int dtype,
                               cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const int cache_row = hidden <= 8192 ? 1 : 0;
  const size_t smem = cache_row ? sizeof(float) * hidden : 0;
  const bool aligned = (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
  if (aligned && num_rows >= NORM_WARP_ROWS && (hidden == 256 || hidden == 512 || hidden == 1024 || hidden == 2048)) {
    if (dtype == TS_DTYPE_F32)
      return launch_add_rms_norm_warp<float>(resid, (const float*)delta, (const float*)weight, (float*)out, rows, num_rows,
                                             hidden, eps, stream);
    if (dtype == TS_DTYPE_BF16)
      return launch_add_rms_norm_warp<bf16>(resid, (const bf16*)delta, (const bf16*)weight, (bf16*)out, rows, num_rows,
                                            hidden, eps, stream);
    return TS_ERR_BAD_ARGUMENT;
  }
  if (cache_row && hidden % 4 == 0 && aligned) {
    const int vthreads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
    if (dtype == TS_DTYPE_F32)
      return launch(add_rms_norm_vec_kernel<float>, num_rows, vthreads, smem, stream, resid, (const float*)delta,
                    (const float*)weight, (float*)out, rows, hidden, eps);
    if (dtype == TS_DTYPE_BF16)
      return launch(add_rms_norm_vec_kernel<bf16>, num_rows, vthreads, smem, stream, resid, (const bf16*)delta,
                    (const bf16*)weight, (bf16*)out, rows, hidden, eps);
    return TS_ERR_BAD_ARGUMENT;
  }
  if (dtype == TS_DTYPE_F32)
    return launch(add_rms_norm_kernel<float>, num_rows, threads, smem, stream, resid, (const float*)delta,
                  (const float*)weight, (float*)out, rows, hidden, eps, cache_row);
  if (dtype == TS_DTYPE_BF16)
    return launch(add_rms_norm_kernel<bf16>, num_rows, threads, smem, stream, resid, (const bf16*)delta,
                  (const bf16*)weight, (bf16*)out, rows, hidden, eps, cache_row);
  return TS_ERR_BAD_ARGUMENT;
}

extern "C" int ts_rope_tables(const int* positions, const double* inv_freq, float* cos_out, float* sin_out,
                              int num_tokens, int half, cudaStream_t stream) {
  const int total = num_tokens * half;
  if (total <= 0) return 0;
  return launch(rope_tables_kernel, (total + 255) / 256, 256, 0, stream, positions, inv_freq, cos_out, sin_out,
                num_tokens, half);
}

extern "C" int ts_silu_mul(const void* gate_up, void* out, int num_tokens, int inter, int dtype,
                           cudaStream_t stream) {
  const size_t total = (size_t)num_tokens * inter;
  if (total == 0) return 0;
  const int vec = dtype == TS_DTYPE_F32 ? 4 : 8;
  if (inter % vec == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
    const size_t total_vecs = total / vec;
    size_t vblocks = (total_vecs + 255) / 256;
    if (vblocks > 148 * 16) vblocks = 148 * 16;
    if (dtype == TS_DTYPE_F32)
      return launch(silu_mul_vec_kernel<float>, (int)vblocks, 256, 0, stream, (const float*)gate_up, (float*)out, inter, total_vecs);
    if (dtype == TS_DTYPE_BF16)
      return launch(silu_mul_vec_kernel<bf16>, (int)vblocks, 256, 0, stream, (const bf16*)gate_up, (bf16*)out, inter, total_vecs);
    return TS_ERR_BAD_ARGUMENT;
  }
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (dtype == TS_DTYPE_F32)
    return launch(silu_mul_kernel<float>, (int)blocks, 256, 0, stream, (const float*)gate_up, (float*)out, inter, total);
  if (dtype == TS_DTYPE_BF16)
    return launch(silu_mul_kernel<bf16>, (int)blocks, 256, 0, stream, (const bf16*)gate_up, (bf16*)out, inter, total);
  return TS_ERR_BAD_ARGUMENT;
}
