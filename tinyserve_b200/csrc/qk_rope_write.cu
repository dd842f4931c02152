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

// The same for many tokens (prefill), bf16, head_dim 64, 128 or 256: D / 16 lanes share a head,
// each with 8 consecutive elements of the first half and their 8 partners of the second (two
// 16-byte accesses), so a warp works on 32 / (D / 16) heads at once and a quarter as many
// instructions move the same bytes as in the kernel above.
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

template <int D>
__global__ void qk_norm_rope_write_wide_kernel(
    const bf16* __restrict__ qkv, bf16* __restrict__ q_out, const bf16* __restrict__ q_weight,
    const bf16* __restrict__ k_weight, float eps, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, const int* __restrict__ slots, bf16* __restrict__ k_cache,
    bf16* __restrict__ v_cache, int page_size, int num_tokens, int num_heads, int num_kv_heads, int write_kv) {
  constexpr int LPH = D / 16, HPW = 32 / LPH, HALF = D / 2;
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPH, l = lane % LPH;
  const int heads_per_token = write_kv ? num_heads + 2 * num_kv_heads : num_heads;
  const long long item = ((long long)blockIdx.x * QK_WARPS + warp) * HPW + sub;
  const bool live = item < (long long)num_tokens * heads_per_token;
  const int t = live ? (int)(item / heads_per_token) : 0;
  const int h = live ? (int)(item - (long long)t * heads_per_token) : 0;
  const bf16* src = qkv + ((size_t)t * heads_per_token + h) * D + 8 * l;
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
  dst += 8 * l;
  uint4 ua = make_uint4(0u, 0u, 0u, 0u), ub = ua;
  if (live) {
    ua = *reinterpret_cast<const uint4*>(src);
    ub = *reinterpret_cast<const uint4*>(src + HALF);
  }
  if (is_v && live) {
    *reinterpret_cast<uint4*>(dst) = ua;
    *reinterpret_cast<uint4*>(dst + HALF) = ub;
  }
  float a[8], b[8];
  unpack8(ua, a);
  unpack8(ub, b);
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss += a[e] * a[e] + b[e] * b[e];
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // within the head's lanes
  if (!live || is_v) return;
  if (weight != nullptr) {
    const float rstd = rsqrtf(ss / (float)D + eps);
    float fa[8], fb[8];
    unpack8(*reinterpret_cast<const uint4*>(weight + 8 * l), fa);
    unpack8(*reinterpret_cast<const uint4*>(weight + HALF + 8 * l), fb);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      a[e] = round_to<bf16>(round_to<bf16>(a[e] * rstd) * fa[e]);
      b[e] = round_to<bf16>(round_to<bf16>(b[e] * rstd) * fb[e]);
    }
  }
  const float* cp = cos_t + (size_t)t * HALF + 8 * l;
  const float* sp = sin_t + (size_t)t * HALF + 8 * l;
  const float4 c0 = *reinterpret_cast<const float4*>(cp), c1 = *reinterpret_cast<const float4*>(cp + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
  const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  float ra[8], rb[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    ra[e] = a[e] * c[e] - b[e] * sn[e];
    rb[e] = b[e] * c[e] + a[e] * sn[e];
  }
  *reinterpret_cast<uint4*>(dst) = pack8(ra);
  *reinterpret_cast<uint4*>(dst + HALF) = pack8(rb);
}

template <int D>
static int launch_wide(const void* qkv, void* q_out, const void* q_weight, const void* k_weight, float eps,
                       const float* cos_t, const float* sin_t, const int* slots, void* k_cache, void* v_cache,
                       int page_size, int num_tokens, int num_heads, int num_kv_heads, int write_kv, cudaStream_t stream) {
  constexpr int HPW = 32 / (D / 16);
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
