// Per-head q/k RMSNorm + rotary position encoding + write of k and v into the paged cache,
// one launch per layer (the upstream engine's fused kernel does the same per (token, head):
// src/tinyserve/triton_fused.py:43-113; formulas src/tinyserve/layers.py:35-38,84-91).
//
// One warp handles one (token, head). q heads: normalise, rotate, write to q_out[t, h, :].
// k heads: normalise, rotate, write to k_cache at the token's slot. v heads: copy to v_cache.
// Norm: 32-bit mean of squares over head_dim, value cast to T, times the weight, rounded to T.
// Rotation in 32-bit on the rounded values, result rounded to T once.
// Cache layout: [page, kv_head, offset_in_page, head_dim]; slot = page * page_size + offset.
#define TS_PDL_CLASS PDL_ELEMENTWISE
#include "common.cuh"

namespace ts {

constexpr int QK_WARPS = 4;
constexpr int QK_MAX_HEAD_DIM = 512;

template <typename T>
__global__ void qk_norm_rope_write_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, const T* __restrict__ q_weight,
    const T* __restrict__ k_weight, float eps, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, int rotary_dim, int interleaved, const int* __restrict__ slots,
    T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, int num_tokens, int num_heads,
    int num_kv_heads, int head_dim, int write_kv) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* buf = smem + warp * head_dim;
  const int heads_per_token = write_kv ? num_heads + 2 * num_kv_heads : num_heads;
  const long long item = (long long)blockIdx.x * QK_WARPS + warp;
  if (item >= (long long)num_tokens * heads_per_token) return;
  const int t = (int)(item / heads_per_token);
  const int h = (int)(item - (long long)t * heads_per_token);
  const T* src = qkv + ((size_t)t * heads_per_token + h) * head_dim;

  // where this head goes
  T* dst;
  const T* weight = nullptr;
  bool rotate = rotary_dim > 0;
  if (h < num_heads) {
    dst = q_out + ((size_t)t * num_heads + h) * head_dim;
    weight = q_weight;
  } else {
    const int slot = slots[t];
    const int page = slot / page_size, off = slot - page * page_size;
    const bool is_k = h < num_heads + num_kv_heads;
    const int kvh = is_k ? h - num_heads : h - num_heads - num_kv_heads;
    T* cache = is_k ? k_cache : v_cache;
    dst = cache + (((size_t)page * num_kv_heads + kvh) * page_size + off) * head_dim;
    if (is_k) {
      weight = k_weight;
    } else {
      for (int i = lane; i < head_dim; i += 32) dst[i] = src[i];
      return;
    }
  }

  // norm (optional)
  if (weight != nullptr) {
    float ss = 0.f;
    for (int i = lane; i < head_dim; i += 32) {
      const float v = to_float(src[i]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)head_dim + eps);
    for (int i = lane; i < head_dim; i += 32) {
      const float n = round_to<T>(to_float(src[i]) * rstd);
      buf[i] = round_to<T>(n * to_float(weight[i]));
    }
  } else {
    for (int i = lane; i < head_dim; i += 32) buf[i] = to_float(src[i]);
  }
  __syncwarp();

  if (!rotate) {
    for (int i = lane; i < head_dim; i += 32) dst[i] = from_float<T>(buf[i]);
    return;
  }
  const int half = rotary_dim >> 1;
  const float* c = cos_t + (size_t)t * half;
  const float* s = sin_t + (size_t)t * half;
  for (int p = lane; p < half; p += 32) {
    const int ia = interleaved ? 2 * p : p;
    const int ib = interleaved ? 2 * p + 1 : p + half;
    const float a = buf[ia], b = buf[ib];
    dst[ia] = from_float<T>(a * c[p] - b * s[p]);
    dst[ib] = from_float<T>(b * c[p] + a * s[p]);
  }
  for (int i = rotary_dim + lane; i < head_dim; i += 32) dst[i] = from_float<T>(buf[i]);
}


// Two adjacent elements with one access (the element index is even, rows are 16-byte aligned).
__device__ __forceinline__ void load2(const float* p, float (&f)[2]) {
  const float2 v = *reinterpret_cast<const float2*>(p);
  f[0] = v.x; f[1] = v.y;
}
__device__ __forceinline__ void load2(const bf16* p, float (&f)[2]) {
  const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
  f[0] = __uint_as_float(w << 16); f[1] = __uint_as_float(w & 0xffff0000u);
}
__device__ __forceinline__ void store2(float* p, const float (&f)[2]) {
  *reinterpret_cast<float2*>(p) = make_float2(f[0], f[1]);
}
__device__ __forceinline__ void store2(bf16* p, const float (&f)[2]) {
  __nv_bfloat162 h = __floats2bfloat162_rn(f[0], f[1]);
  *reinterpret_cast<uint32_t*>(p) = *reinterpret_cast<uint32_t*>(&h);
}

// Register-only variant for the common case: the whole head is rotated with the "half" pairing
// (rotary_dim == head_dim, head_dim % 4 == 0). A lane owns pairs p = 2 lane, 2 lane + 1 (+ 64 j):
// elements p, p + 1 and their partners p + D/2, p + 1 + D/2, each fetched with one access.
template <typename T, int MAXJ>
__global__ void qk_norm_rope_write_fast_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, const T* __restrict__ q_weight,
    const T* __restrict__ k_weight, float eps, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, const int* __restrict__ slots, T* __restrict__ k_cache,
    T* __restrict__ v_cache, int page_size, int num_tokens, int num_heads, int num_kv_heads, int head_dim,
    int write_kv) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_per_token = write_kv ? num_heads + 2 * num_kv_heads : num_heads;
  const long long item = (long long)blockIdx.x * QK_WARPS + warp;
  if (item >= (long long)num_tokens * heads_per_token) return;
  const int t = (int)(item / heads_per_token);
  const int h = (int)(item - (long long)t * heads_per_token);
  const T* src = qkv + ((size_t)t * heads_per_token + h) * head_dim;
  T* dst;
  const T* weight = nullptr;
  if (h < num_heads) {
    dst = q_out + ((size_t)t * num_heads + h) * head_dim;
    weight = q_weight;
  } else {
    const int slot = slots[t];
    const int page = slot / page_size, off = slot - page * page_size;
    const bool is_k = h < num_heads + num_kv_heads;
    const int kvh = is_k ? h - num_heads : h - num_heads - num_kv_heads;
    dst = (is_k ? k_cache : v_cache) + (((size_t)page * num_kv_heads + kvh) * page_size + off) * head_dim;
    if (!is_k) {
      constexpr int VEC = Vec<T>::N;
      for (int i = lane * VEC; i < head_dim; i += 32 * VEC) {
        Vec<T> v;
        v.load(src + i);
        v.store(dst + i);
      }
      return;
    }
    weight = k_weight;
  }
  const int half = head_dim >> 1;
  float a[MAXJ][2], b[MAXJ][2];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXJ; ++j) {
    const int p = 2 * lane + 64 * j;
    a[j][0] = a[j][1] = b[j][0] = b[j][1] = 0.f;
    if (p < half) {
      load2(src + p, a[j]);
      load2(src + half + p, b[j]);
      ss += a[j][0] * a[j][0] + a[j][1] * a[j][1] + b[j][0] * b[j][0] + b[j][1] * b[j][1];
    }
  }
  if (weight != nullptr) {
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)head_dim + eps);
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int p = 2 * lane + 64 * j;
      if (p < half) {
        float wa[2], wb[2];
        load2(weight + p, wa);
        load2(weight + half + p, wb);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          a[j][e] = round_to<T>(round_to<T>(a[j][e] * rstd) * wa[e]);
          b[j][e] = round_to<T>(round_to<T>(b[j][e] * rstd) * wb[e]);
        }
      }
    }
  }
  const float* c = cos_t + (size_t)t * half;
  const float* s = sin_t + (size_t)t * half;
#pragma unroll
  for (int j = 0; j < MAXJ; ++j) {
    const int p = 2 * lane + 64 * j;
    if (p < half) {
      const float2 cv = *reinterpret_cast<const float2*>(c + p);
      const float2 sv = *reinterpret_cast<const float2*>(s + p);
      const float ra[2] = {a[j][0] * cv.x - b[j][0] * sv.x, a[j][1] * cv.y - b[j][1] * sv.y};
      const float rb[2] = {b[j][0] * cv.x + a[j][0] * sv.x, b[j][1] * cv.y + a[j][1] * sv.y};
      store2(dst + p, ra);
      store2(dst + half + p, rb);
    }
  }
}

// The same for many tokens (prefill), bf16, head_dim 64, 128 or 256: D / 8 lanes share a head,
// each with 4 consecutive elements of the first half and their 4 partners of the second (two
// 8-byte accesses), so a warp works on 32 / (D / 8) heads at once and half as many instructions
// move the same bytes as in the kernel above.
template <int D>
__global__ void qk_norm_rope_write_wide_kernel(
    const bf16* __restrict__ qkv, bf16* __restrict__ q_out, const bf16* __restrict__ q_weight,
    const bf16* __restrict__ k_weight, float eps, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, const int* __restrict__ slots, bf16* __restrict__ k_cache,
    bf16* __restrict__ v_cache, int page_size, int num_tokens, int num_heads, int num_kv_heads, int write_kv) {
  constexpr int LPH = D / 8, HPW = 32 / LPH, HALF = D / 2;
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPH, l = lane % LPH;
  const int heads_per_token = write_kv ? num_heads + 2 * num_kv_heads : num_heads;
  const long long item = ((long long)blockIdx.x * QK_WARPS + warp) * HPW + sub;
  const bool live = item < (long long)num_tokens * heads_per_token;
  const int t = live ? (int)(item / heads_per_token) : 0;
  const int h = live ? (int)(item - (long long)t * heads_per_token) : 0;
  const bf16* src = qkv + ((size_t)t * heads_per_token + h) * D + 4 * l;
  bf16* dst;
  const bf16* weight = nullptr;
  bool is_v = false;
  if (h < num_heads) {
    dst = q_out + ((size_t)t * num_heads + h) * D;
    weight = q_weight;
  } else {
    const int slot = slots[t];
    const int page = slot / page_size, off = slot - page * page_size;
    const bool is_k = h < num_heads + num_kv_heads;
    const int kvh = is_k ? h - num_heads : h - num_heads - num_kv_heads;
    dst = (is_k ? k_cache : v_cache) + (((size_t)page * num_kv_heads + kvh) * page_size + off) * D;
    is_v = !is_k;
    weight = k_weight;
  }
  dst += 4 * l;
  uint2 ua = make_uint2(0u, 0u), ub = make_uint2(0u, 0u);
  if (live) {
    ua = *reinterpret_cast<const uint2*>(src);
    ub = *reinterpret_cast<const uint2*>(src + HALF);
  }
  if (is_v) {
    if (live) {
      *reinterpret_cast<uint2*>(dst) = ua;
      *reinterpret_cast<uint2*>(dst + HALF) = ub;
    }
  }
  float a[4] = {__uint_as_float(ua.x << 16), __uint_as_float(ua.x & 0xffff0000u), __uint_as_float(ua.y << 16),
                __uint_as_float(ua.y & 0xffff0000u)};
  float b[4] = {__uint_as_float(ub.x << 16), __uint_as_float(ub.x & 0xffff0000u), __uint_as_float(ub.y << 16),
                __uint_as_float(ub.y & 0xffff0000u)};
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) ss += a[e] * a[e] + b[e] * b[e];
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // within the head's lanes
  if (!live || is_v) return;
  if (weight != nullptr) {
    const float rstd = rsqrtf(ss / (float)D + eps);
    const uint2 wa = *reinterpret_cast<const uint2*>(weight + 4 * l);
    const uint2 wb = *reinterpret_cast<const uint2*>(weight + HALF + 4 * l);
    const float fa[4] = {__uint_as_float(wa.x << 16), __uint_as_float(wa.x & 0xffff0000u), __uint_as_float(wa.y << 16),
                         __uint_as_float(wa.y & 0xffff0000u)};
    const float fb[4] = {__uint_as_float(wb.x << 16), __uint_as_float(wb.x & 0xffff0000u), __uint_as_float(wb.y << 16),
                         __uint_as_float(wb.y & 0xffff0000u)};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      a[e] = round_to<bf16>(round_to<bf16>(a[e] * rstd) * fa[e]);
      b[e] = round_to<bf16>(round_to<bf16>(b[e] * rstd) * fb[e]);
    }
  }
  const float4 cv = *reinterpret_cast<const float4*>(cos_t + (size_t)t * HALF + 4 * l);
  const float4 sv = *reinterpret_cast<const float4*>(sin_t + (size_t)t * HALF + 4 * l);
  const float c[4] = {cv.x, cv.y, cv.z, cv.w}, sn[4] = {sv.x, sv.y, sv.z, sv.w};
  float ra[4], rb[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    ra[e] = a[e] * c[e] - b[e] * sn[e];
    rb[e] = b[e] * c[e] + a[e] * sn[e];
  }
  __nv_bfloat162 p0 = __floats2bfloat162_rn(ra[0], ra[1]), p1 = __floats2bfloat162_rn(ra[2], ra[3]);
  __nv_bfloat162 q0 = __floats2bfloat162_rn(rb[0], rb[1]), q1 = __floats2bfloat162_rn(rb[2], rb[3]);
  *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1));
  *reinterpret_cast<uint2*>(dst + HALF) = make_uint2(*reinterpret_cast<uint32_t*>(&q0), *reinterpret_cast<uint32_t*>(&q1));
}

template <int D>
static int launch_wide(const void* qkv, void* q_out, const void* q_weight, const void* k_weight, float eps,
                       const float* cos_t, const float* sin_t, const int* slots, void* k_cache, void* v_cache,
                       int page_size, int num_tokens, int num_heads, int num_kv_heads, int write_kv, cudaStream_t stream) {
  constexpr int HPW = 32 / (D / 8);
  const int heads_per_token = write_kv ? num_heads + 2 * num_kv_heads : num_heads;
  const long long items = (long long)num_tokens * heads_per_token;
  const long long per_block = (long long)QK_WARPS * HPW;
  return launch(qk_norm_rope_write_wide_kernel<D>, (int)((items + per_block - 1) / per_block), QK_WARPS * 32, 0, stream,
                (const bf16*)qkv, (bf16*)q_out, (const bf16*)q_weight, (const bf16*)k_weight, eps, cos_t, sin_t, slots,
                (bf16*)k_cache, (bf16*)v_cache, page_size, num_tokens, num_heads, num_kv_heads, write_kv);
}

}  // namespace ts

using namespace ts;

extern "C" int ts_qk_norm_rope_write(const void* qkv, void* q_out, const void* q_weight, const void* k_weight,
                                     float eps, const float* cos_t, const float* sin_t, int rotary_dim,
                                     int interleaved, const int* slots, void* k_cache, void* v_cache,
                                     int page_size, int num_tokens, int num_heads, int num_kv_heads,
                                     int head_dim, int write_kv, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (head_dim <= 0 || head_dim > QK_MAX_HEAD_DIM || rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1))
    return TS_ERR_UNSUPPORTED;
  const int heads_per_token = write_kv ? num_heads + 2 * num_kv_heads : num_heads;
  const long long items = (long long)num_tokens * heads_per_token;
  const int blocks = (int)((items + QK_WARPS - 1) / QK_WARPS);
  const size_t smem = (size_t)QK_WARPS * head_dim * sizeof(float);
  if (rotary_dim == head_dim && !interleaved && head_dim % 8 == 0 && head_dim <= 256 &&
      (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0) {
    if (dtype == TS_DTYPE_BF16 && num_tokens >= 32 && (q_weight == nullptr) == (k_weight == nullptr)) {
#define TS_WIDE(D_)                                                                                              \
  return launch_wide<D_>(qkv, q_out, q_weight, k_weight, eps, cos_t, sin_t, slots, k_cache, v_cache, page_size, \
                         num_tokens, num_heads, num_kv_heads, write_kv, stream)
      if (head_dim == 64) { TS_WIDE(64); }
      if (head_dim == 128) { TS_WIDE(128); }
      if (head_dim == 256) { TS_WIDE(256); }
#undef TS_WIDE
    }
    if (dtype == TS_DTYPE_F32)
      return launch(qk_norm_rope_write_fast_kernel<float, 2>, blocks, QK_WARPS * 32, 0, stream,
                    (const float*)qkv, (float*)q_out, (const float*)q_weight, (const float*)k_weight, eps, cos_t,
                    sin_t, slots, (float*)k_cache, (float*)v_cache, page_size, num_tokens, num_heads, num_kv_heads,
                    head_dim, write_kv);
    if (dtype == TS_DTYPE_BF16)
      return launch(qk_norm_rope_write_fast_kernel<bf16, 2>, blocks, QK_WARPS * 32, 0, stream,
                    (const bf16*)qkv, (bf16*)q_out, (const bf16*)q_weight, (const bf16*)k_weight, eps, cos_t,
                    sin_t, slots, (bf16*)k_cache, (bf16*)v_cache, page_size, num_tokens, num_heads, num_kv_heads,
                    head_dim, write_kv);
    return TS_ERR_BAD_ARGUMENT;
  }
  if (dtype == TS_DTYPE_F32)
    return launch(qk_norm_rope_write_kernel<float>, blocks, QK_WARPS * 32, smem, stream,
        (const float*)qkv, (float*)q_out, (const float*)q_weight, (const float*)k_weight, eps, cos_t, sin_t,
        rotary_dim, interleaved, slots, (float*)k_cache, (float*)v_cache, page_size, num_tokens, num_heads,
        num_kv_heads, head_dim, write_kv);
  if (dtype == TS_DTYPE_BF16)
    return launch(qk_norm_rope_write_kernel<bf16>, blocks, QK_WARPS * 32, smem, stream,
        (const bf16*)qkv, (bf16*)q_out, (const bf16*)q_weight, (const bf16*)k_weight, eps, cos_t, sin_t,
        rotary_dim, interleaved, slots, (bf16*)k_cache, (bf16*)v_cache, page_size, num_tokens, num_heads,
        num_kv_heads, head_dim, write_kv);
  return TS_ERR_BAD_ARGUMENT;
}
