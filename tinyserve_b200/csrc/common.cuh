// Shared helpers of the sm_100a kernels: element types, 16-byte vector access, reductions.
// Every kernel is instantiated for float (the true 32-bit path) and __nv_bfloat16.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TS_DTYPE_F32 0
#define TS_DTYPE_BF16 1

// Error codes returned by the extern "C" launchers (0 = ok, >0 = cudaError_t).
#define TS_ERR_BAD_ARGUMENT (-1)
#define TS_ERR_UNSUPPORTED (-2)

namespace ts {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float x) { return __float2bfloat16_rn(x); }

// Round a 32-bit value to the storage type and back: the rounding points of the model.
template <typename T> __device__ __forceinline__ float round_to(float x) { return to_float(from_float<T>(x)); }

// 16-byte vectors: VEC elements of T.
template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = raw; }
  __device__ __forceinline__ void zero() { raw = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ void unpack(float* f) const { f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w; }
  __device__ __forceinline__ void pack(const float* f) { raw = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec<bf16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ void load(const bf16* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(bf16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ void zero() { raw = make_uint4(0u, 0u, 0u, 0u); }
  __device__ __forceinline__ void unpack(float* f) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // bf16 -> f32 is a 16-bit shift.
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ void pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    raw = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// "The CTA that arrives last does the merge": every CTA of a group calls this after writing its
// partial results; it returns true in exactly one of them, the last to arrive, after which that
// CTA may read all partial results (with __ldcg). The barrier orders the CTA's writes before
// thread 0's release, and thread 0's acquire before the CTA's later reads. The counter is put
// back to zero by the last arriver, so it never needs clearing between launches.
__device__ __forceinline__ bool cta_arrives_last(unsigned int* counter, unsigned int group_size, int* flag_in_smem) {
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
    const int last = (old == group_size - 1u);
    if (last) *counter = 0u;
    *flag_in_smem = last;
  }
  __syncthreads();
  return *flag_in_smem != 0;
}

static inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return (int)e;
}

// ---- programmatic dependent launch
// Kernels of one step form a chain on one stream. When this switch is on they are launched so
// that the next kernel's CTAs may be scheduled while the previous kernel is still draining:
// every kernel calls pdl_trigger() at its start and pdl_wait() before it reads anything an
// earlier kernel wrote or writes anything at all. pdl_wait() returns once every earlier kernel
// of the chain has finished and its writes are visible, so ordering is what it was; only the
// launch latency and the part of a kernel that needs no input (index arithmetic, prefetch of
// weights) overlap the predecessor. Off, the two calls do nothing.
// The switch is a mask of kernel classes, so that the overlap can be limited to the kernels that
// gain from it.
extern int g_programmatic_launch;   // defined in elementwise.cu, set by ts_set_programmatic_launch
constexpr int PDL_ELEMENTWISE = 1, PDL_SKINNY = 2, PDL_ATTENTION = 4, PDL_TCGEN05 = 8, PDL_SAMPLING = 16, PDL_OTHER = 32;
#ifndef TS_PDL_CLASS
#define TS_PDL_CLASS PDL_OTHER
#endif

#ifdef TS_TIMELINE
// Built with -DTS_TIMELINE, the first thread of the first CTA of every launch notes the device
// clock (ns) when it starts and when its wait for the earlier kernels returns: the only way to
// see, inside a replayed graph with overlapping launches, when each kernel really began and how
// long the chain before it took. Records are kept per source file and read back sorted by time
// (ts_timeline_read). Costs an atomic and two stores per launch; never part of a timed build.
constexpr int TL_CAP = 16384;
static __device__ unsigned long long tl_records[TL_CAP * 3];
static __device__ unsigned int tl_count;
extern "C" void ts_timeline_register(void* records, void* count, int cap);
__device__ __forceinline__ unsigned long long tl_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned int& tl_slot() {
  __shared__ unsigned int slot;
  return slot;
}
__device__ __forceinline__ bool tl_first() {
  return (threadIdx.x | threadIdx.y | threadIdx.z | blockIdx.x | blockIdx.y | blockIdx.z) == 0;
}
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (tl_first()) {
    const unsigned int s = atomicAdd(&tl_count, 1u) % TL_CAP;
    tl_slot() = s;
    tl_records[3 * s] = (unsigned long long)TS_PDL_CLASS | ((unsigned long long)gridDim.x << 8) |
                        ((unsigned long long)gridDim.y << 28) | ((unsigned long long)blockDim.x << 44);
    tl_records[3 * s + 2] = 0;
    tl_records[3 * s + 1] = tl_now();
  }
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (tl_first()) {
    const unsigned int s = tl_slot();
    if (tl_records[3 * s + 2] == 0) tl_records[3 * s + 2] = tl_now();
  }
}
static inline void tl_register_once() {
  static bool done = false;
  if (done) return;
  done = true;
  void *r = nullptr, *c = nullptr;
  if (cudaGetSymbolAddress(&r, tl_records) == cudaSuccess && cudaGetSymbolAddress(&c, tl_count) == cudaSuccess)
    ts_timeline_register(r, c, TL_CAP);
}
#else
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
static inline void tl_register_once() {}
#endif

template <typename... KArgs, typename... Args>
static inline int launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                         Args... args) {
  tl_register_once();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (g_programmatic_launch & TS_PDL_CLASS) ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the CTAs grouped into thread-block clusters of `cluster` CTAs.
template <typename... KArgs, typename... Args>
static inline int launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 dim3 cluster, Args... args) {
  tl_register_once();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (g_programmatic_launch & TS_PDL_CLASS) ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace ts
