// out[M, N] = x[M, K] * w[N, K]^T in bf16 on the 5th-generation tensor cores: TMA loads into
// 128-byte-swizzled shared memory, tcgen05.mma issued by one thread with the accumulator in
// tensor memory (TMEM), tcgen05.ld for the epilogue. bf16 or float output from the 32-bit
// accumulator. The library product that this replaces is upstream's F.linear
// (src/tinyserve/model.py:156,173,178-179,208).
//
// A CTA computes 128 x BN tiles, one after the other. Both operands are K-major in memory ([rows, K] row-major),
// which is the layout the instruction wants, so a stage is two TMA boxes: 128 rows x 64 k of x
// and BN rows x 64 k of w. Out-of-range rows and the K tail read as zeros (TMA fill), so any
// M, N and any K that is a multiple of 8 (16-byte row pitch) are taken.
//   warp 0, one lane : TMA producer        (waits "empty", arms "full" with the byte count)
//   warp 1, one lane : MMA issuer          (waits "full", 4 x tcgen05.mma of K = 16 per stage,
//                                           tcgen05.commit frees the stage; last commit of a tile
//                                           marks its accumulator "full")
//   warps 2-5        : epilogue            (tcgen05.ld of the warp's 32 TMEM lanes, cast, store,
//                                           then the accumulator buffer is handed back)
// SWIGLU variant: w holds 2 N rows (gate rows, then up rows); a tile's B operand is 128 gate
// rows followed by the 128 up rows of the same output columns (two TMA boxes), so the
// accumulator holds gate in columns 0..127 and up in 128..255 and the epilogue writes
// silu(gate) * up, [M, N], with the rounding points of the separate kernels (each product to
// bf16, the SiLU to bf16, the result to bf16; upstream src/tinyserve/layers.py:94-115).
// Every wait on an mbarrier is bounded: when the bound is hit the kernel records it in
// *error_flag, stops waiting and still frees its tensor memory, so a fault in the pipeline
// shows as an error code on the host and never as a hang.
#define TS_PDL_CLASS PDL_TCGEN05
#include <cuda.h>

#include "tcgen05.cuh"

namespace ts {

constexpr int TG_BM = 128;
constexpr int TG_BK = 64;              // 64 bf16 = 128 bytes = one swizzle row
constexpr int TG_THREADS = 192;     // TMA warp, MMA warp, four epilogue warps

// One warp's share of an accumulator tile (its 32 tensor-memory lanes = 32 rows, BN columns from
// tmem_acc) -> out: cast and store, or silu(gate) * up of the two halves (SWIGLU).
template <int BN, typename TOut, bool SWIGLU>
__device__ __forceinline__ void drain_tile(uint32_t tmem_acc, int row, int M, int N, int n0, TOut* __restrict__ out) {
  constexpr int BN_OUT = SWIGLU ? BN / 2 : BN;
  if constexpr (SWIGLU) {
#pragma unroll 1
    for (int c = 0; c < BN_OUT / 32; ++c) {
      uint32_t g[32], u[32];
      const uint32_t base = tmem_acc + (uint32_t)(c * 32);
      tmem_ld_32_nowait(base, g);
      tmem_ld_32_nowait(base + BN_OUT, u);
      tmem_ld_wait();
      if (row < M) {
        bf16* dst = (bf16*)out + (size_t)row * N + n0 + c * 32;
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float gv = round_to<bf16>(__uint_as_float(g[j])), uv = round_to<bf16>(__uint_as_float(u[j]));
          f[j] = round_to<bf16>(__fdividef(gv, 1.f + __expf(-gv))) * uv;
        }
        if (n0 + c * 32 + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            Vec<bf16> v;
            v.pack(f + j);
            v.store(dst + j);
          }
        } else {
          for (int j = 0; j < 32; ++j)
            if (n0 + c * 32 + j < N) dst[j] = from_float<bf16>(f[j]);
        }
      }
    }
  } else {
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32(tmem_acc + (uint32_t)(c * 32), r);
    if (row < M) {
      TOut* dst = out + (size_t)row * N + n0 + c * 32;
      if (n0 + c * 32 + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
        if constexpr (sizeof(TOut) == 2) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[j + e]);
            Vec<bf16> v;
            v.pack(f);
            v.store((bf16*)dst + j);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>((float*)dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                                    __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        }
      } else {
        for (int j = 0; j < 32; ++j)
          if (n0 + c * 32 + j < N) dst[j] = from_float<TOut>(__uint_as_float(r[j]));
      }
    }
  }
  }
}

// Persistent, warp-specialised: a CTA loops over output tiles (tile = blockIdx.x + i * gridDim.x,
// rows fastest, so CTAs that run together share weight tiles in L2). The accumulator is double-
// buffered in tensor memory (2 x BN columns): while the four epilogue warps drain tile i, the
// MMA warp already accumulates tile i + 1.
template <int BN, int STAGES, typename TOut, bool SWIGLU = false>
__global__ void __launch_bounds__(TG_THREADS) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                  const __grid_constant__ CUtensorMap map_w,
                                                                  TOut* __restrict__ out, int M, int N, int K,
                                                                  int* __restrict__ error_flag) {
  constexpr uint32_t A_BYTES = TG_BM * TG_BK * 2, B_BYTES = BN * TG_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  // instruction descriptor: D = f32, A = B = bf16, both K-major, N = BN, M = 128
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TG_BM >> 4) << 24);
  constexpr uint32_t TMEM_COLS = 2 * BN;      // a power of two >= 32: BN in {64, 128, 256}
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  static_assert(!SWIGLU || BN == 256, "the fused activation pairs 128 gate with 128 up columns");
  constexpr int BN_OUT = SWIGLU ? BN / 2 : BN;          // output columns per tile
  const int tiles_m = (M + TG_BM - 1) / TG_BM, tiles_n = (N + BN_OUT - 1) / BN_OUT;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + TG_BK - 1) / TG_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ---------------- TMA producer (one lane)
    if (lane == 0 && !wait_test_unarmed()) {
      // The weights do not depend on the kernel before this one: the B tiles of the first stages
      // are requested before the wait for it, the A tiles (its output) after.
      auto load_b = [&](int s, int kb, int n0) {
        unsigned char* a = tiles + (size_t)s * STAGE_BYTES;
        if constexpr (SWIGLU) {
          // the map's box is 128 rows: gate rows n0.., then up rows N + n0.. of the merged matrix
          tma_load_2d(a + A_BYTES, &map_w, &full_bar[s], kb * TG_BK, n0);
          tma_load_2d(a + A_BYTES + B_BYTES / 2, &map_w, &full_bar[s], kb * TG_BK, N + n0);
        } else {
          tma_load_2d(a + A_BYTES, &map_w, &full_bar[s], kb * TG_BK, n0);
        }
      };
      int early = 0;
      if ((int)blockIdx.x < num_tiles) {
        const int n0 = ((int)blockIdx.x / tiles_m) * BN_OUT;
        early = num_kb < STAGES ? num_kb : STAGES;
        for (int kb = 0; kb < early; ++kb) {          // fresh barriers: nothing to wait for
          mbar_expect_tx(&full_bar[kb], STAGE_BYTES);
          load_b(kb, kb, n0);
        }
      }
      pdl_wait();
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !failed; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * TG_BM, n0 = (tile / tiles_m) * BN_OUT;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          unsigned char* a = tiles + (size_t)s * STAGE_BYTES;
          if (it >= early) {
            if (!mbar_wait(&empty_bar[s], phase ^ 1)) { failed = 1; break; }
            mbar_expect_tx(&full_bar[s], STAGE_BYTES);
            load_b(s, kb, n0);
          }
          tma_load_2d(a, &map_x, &full_bar[s], kb * TG_BK, m0);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (one lane)
    if (lane == 0) {
      int it = 0, t = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !failed; tile += gridDim.x, ++t) {
        const int b = t & 1;
        // the epilogue must have drained this accumulator (two tiles ago)
        if (!mbar_wait(&acc_empty[b], ((t >> 1) & 1) ^ 1)) { failed = 1; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], phase)) { failed = 1; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint64_t adesc = sw128_desc(a_addr), bdesc = sw128_desc(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < TG_BK / 16; ++k) {
            // 16 k = 32 bytes further along the swizzled row: +2 in the descriptor's 16-byte units
            umma_bf16(tmem_d, adesc + 2 * k, bdesc + 2 * k, IDESC, (kb | k) != 0);
          }
          umma_commit(&empty_bar[s]);   // the stage is free once these MMAs have read it
        }
        umma_commit(&acc_full[b]);      // the accumulator is complete once every MMA has finished
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5; warp w may touch TMEM lanes 32 (w % 4) .. + 31
    pdl_wait();      // out may be written only once the kernel before this one is done
    const int quad = warp & 3;
    int t = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
      const int b = t & 1;
      const int m0 = (tile % tiles_m) * TG_BM, n0 = (tile / tiles_m) * BN_OUT;
      if (!mbar_wait(&acc_full[b], (t >> 1) & 1) || failed) {
        if (lane == 0) atomicExch(error_flag, WAIT_FAILED_GEMM_TCGEN05);
        break;
      }
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      drain_tile<BN, TOut, SWIGLU>(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(b * BN), row, M, N, n0, out);
      // this warp has read its part of the accumulator: hand the buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// The same product by pairs of CTAs (clusters of two, tcgen05 cta_group::2): a pair computes 256 x 256
// tiles. Each CTA loads its 128 rows of x and its half of the tile's 256 rows of w (SWIGLU: the even
// CTA the 128 gate rows, the odd one the 128 up rows), so a CTA fetches 32 KB per 64 k where the
// single-CTA kernel fetches 48 KB for half the work: a third less traffic from L2 per flop, and six
// stages instead of four in the same shared memory. One thread of the even CTA issues the MMAs for
// both (M = 256: rows 0..127 accumulate in the even CTA's tensor memory, 128..255 in the odd one's);
// its commits arrive at the barriers of both CTAs; both CTAs' TMA copies report their bytes to the
// even CTA's "full" barrier; each CTA's epilogue warps drain their own tensor memory and hand the
// accumulator back to the even CTA's MMA thread.
template <int STAGES, typename TOut, bool SWIGLU>
__global__ void __launch_bounds__(TG_THREADS) gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                       const __grid_constant__ CUtensorMap map_w,
                                                                       TOut* __restrict__ out, int M, int N, int K,
                                                                       int* __restrict__ error_flag) {
  constexpr int BN = 256, PAIR_BM = 2 * TG_BM;
  constexpr uint32_t A_BYTES = TG_BM * TG_BK * 2, B_BYTES = (BN / 2) * TG_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;   // per CTA
  // instruction descriptor: D = f32, A = B = bf16, both K-major, N = 256, M = 256 over the pair
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(PAIR_BM >> 4) << 24);
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr int BN_OUT = SWIGLU ? BN / 2 : BN;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];      // used in the even CTA: the bytes of both CTAs' copies
  __shared__ __align__(8) uint64_t empty_bar[STAGES];     // in each CTA: the MMAs have read this stage
  __shared__ __align__(8) uint64_t acc_full[2];           // in each CTA: the accumulator is complete
  __shared__ __align__(8) uint64_t acc_empty[2];          // used in the even CTA: 2 x 4 epilogue warps are done with it
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + PAIR_BM - 1) / PAIR_BM, tiles_n = (N + BN_OUT - 1) / BN_OUT;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + TG_BK - 1) / TG_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(&tmem_base_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // both CTAs' barriers and tensor memory exist before either uses the other's
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t full0 = smem_of_cta(&full_bar[0], 0), acc_empty0 = smem_of_cta(&acc_empty[0], 0);

  if (warp == 0) {
    // ---------------- TMA producer (one lane in each CTA)
    if (lane == 0 && !wait_test_unarmed()) {
      auto load_b = [&](int s, int kb, int n0) {
        const int w_row = SWIGLU ? (leader ? n0 : N + n0) : n0 + (int)rank * (BN / 2);
        tma_load_2d_pair(tiles + (size_t)s * STAGE_BYTES + A_BYTES, &map_w, full0 + 8u * s, kb * TG_BK, w_row);
      };
      // the weights do not depend on the kernel before this one (see gemm_tcgen05_kernel)
      int early = 0;
      if (pair < num_tiles) {
        const int n0 = (pair / tiles_m) * BN_OUT;
        early = num_kb < STAGES ? num_kb : STAGES;
        for (int kb = 0; kb < early; ++kb) {
          if (leader) mbar_expect_tx(&full_bar[kb], 2 * STAGE_BYTES);
          load_b(kb, kb, n0);
        }
      }
      pdl_wait();
      int it = 0;
      for (int tile = pair; tile < num_tiles && !failed; tile += num_pairs) {
        const int m0 = (tile % tiles_m) * PAIR_BM + (int)rank * TG_BM, n0 = (tile / tiles_m) * BN_OUT;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (it >= early) {
            if (!mbar_wait(&empty_bar[s], phase ^ 1)) { failed = 1; break; }
            if (leader) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
            load_b(s, kb, n0);
          }
          tma_load_2d_pair(tiles + (size_t)s * STAGE_BYTES, &map_x, full0 + 8u * s, kb * TG_BK, m0);
        }
      }
      // the even CTA's last commits also arrive at this CTA's barriers: stay until they have
      for (int j = it > STAGES ? it - STAGES : 0; j < it && !failed; ++j)
        if (!mbar_wait(&empty_bar[j % STAGES], (j / STAGES) & 1)) failed = 1;
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (one lane of the even CTA)
    if (lane == 0 && leader) {
      int it = 0, t = 0;
      for (int tile = pair; tile < num_tiles && !failed; tile += num_pairs, ++t) {
        const int b = t & 1;
        if (!mbar_wait(&acc_empty[b], ((t >> 1) & 1) ^ 1)) { failed = 1; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], phase)) { failed = 1; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint64_t adesc = sw128_desc(a_addr), bdesc = sw128_desc(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < TG_BK / 16; ++k) umma_bf16_pair(tmem_d, adesc + 2 * k, bdesc + 2 * k, IDESC, (kb | k) != 0);
          umma_commit_pair(&empty_bar[s]);
        }
        umma_commit_pair(&acc_full[b]);
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 of each CTA drain their own CTA's tensor memory
    pdl_wait();
    const int quad = warp & 3;
    int t = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++t) {
      const int b = t & 1;
      const int m0 = (tile % tiles_m) * PAIR_BM + (int)rank * TG_BM, n0 = (tile / tiles_m) * BN_OUT;
      if (!mbar_wait(&acc_full[b], (t >> 1) & 1) || failed) {
        if (lane == 0) atomicExch(error_flag, WAIT_FAILED_GEMM_TCGEN05);
        break;
      }
      tc_fence_after();
      drain_tile<BN, TOut, SWIGLU>(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(b * BN), m0 + quad * 32 + lane, M, N,
                                   n0, out);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty0 + 8u * b);
    }
  }
  // neither CTA may leave, or free its tensor memory, while the other can still reach it
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// rows x K bf16 row-major; box = box_rows x 64, 128-byte swizzle, zero fill outside.
static bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {(cuuint32_t)TG_BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int STAGES, typename TOut, bool SWIGLU = false>
static int launch_tc(const CUtensorMap& mx, const CUtensorMap& mw, TOut* out, int M, int N, int K, int* error_flag,
                     cudaStream_t stream) {
  const size_t smem = (size_t)STAGES * (TG_BM + BN) * TG_BK * 2 + 1024;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, TOut, SWIGLU>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  constexpr int BN_OUT = SWIGLU ? BN / 2 : BN;
  const int num_tiles = ((N + BN_OUT - 1) / BN_OUT) * ((M + TG_BM - 1) / TG_BM);
  const int ctas = num_tiles < 148 ? num_tiles : 148;     // one persistent CTA per SM
  return launch(kern, ctas, TG_THREADS, smem, stream, mx, mw, out, M, N, K, error_flag);
}

template <int STAGES, typename TOut, bool SWIGLU>
static int launch_tc_pair(const CUtensorMap& mx, const CUtensorMap& mw, TOut* out, int M, int N, int K, int* error_flag,
                          cudaStream_t stream) {
  const size_t smem = (size_t)STAGES * (TG_BM + 128) * TG_BK * 2 + 1024;
  auto kern = gemm_tcgen05_pair_kernel<STAGES, TOut, SWIGLU>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  constexpr int BN_OUT = SWIGLU ? 128 : 256;
  const int num_tiles = ((N + BN_OUT - 1) / BN_OUT) * ((M + 2 * TG_BM - 1) / (2 * TG_BM));
  const int pairs = num_tiles < 74 ? num_tiles : 74;      // one persistent CTA per SM, two SMs a pair
  return launch_cluster(kern, dim3(2 * pairs), dim3(TG_THREADS), smem, stream, dim3(2, 1, 1), mx, mw, out, M, N, K, error_flag);
}

}  // namespace ts

using namespace ts;

// error_flag: device int that the kernel sets to 1 if a bounded wait ran out.
extern "C" int ts_gemm_tcgen05(const void* x, const void* w, void* out, int M, int N, int K, int out_dtype,
                               int tile_n, int* error_flag, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || error_flag == nullptr) return TS_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return TS_ERR_UNSUPPORTED;
  if (tile_n != 64 && tile_n != 128 && tile_n != 256 && tile_n != 512) return TS_ERR_BAD_ARGUMENT;
  CUtensorMap mx, mw;
  if (tile_n == 512) {      // 256 x 256 tiles by pairs of CTAs
    if (!make_map(&mx, x, M, K, TG_BM) || !make_map(&mw, w, N, K, 128)) return TS_ERR_UNSUPPORTED;
    if (out_dtype == TS_DTYPE_F32) return launch_tc_pair<6, float, false>(mx, mw, (float*)out, M, N, K, error_flag, stream);
    if (out_dtype == TS_DTYPE_BF16) return launch_tc_pair<6, bf16, false>(mx, mw, (bf16*)out, M, N, K, error_flag, stream);
    return TS_ERR_BAD_ARGUMENT;
  }
  if (!make_map(&mx, x, M, K, TG_BM) || !make_map(&mw, w, N, K, tile_n)) return TS_ERR_UNSUPPORTED;
  const bool f32 = out_dtype == TS_DTYPE_F32;
  if (!f32 && out_dtype != TS_DTYPE_BF16) return TS_ERR_BAD_ARGUMENT;
#define TS_TC(BN_, ST_)                                                                               \
  return f32 ? launch_tc<BN_, ST_, float>(mx, mw, (float*)out, M, N, K, error_flag, stream)           \
             : launch_tc<BN_, ST_, bf16>(mx, mw, (bf16*)out, M, N, K, error_flag, stream)
  if (tile_n == 64) { TS_TC(64, 6); }
  if (tile_n == 128) { TS_TC(128, 6); }
  TS_TC(256, 4);
#undef TS_TC
}

// act[M, inter] = silu(x gate^T) * (x up^T) in bf16 with w = [gate rows; up rows], [2 inter, K]:
// the product and the activation in one kernel (SWIGLU above). K % 8 == 0.
extern "C" int ts_gemm_tcgen05_swiglu(const void* x, const void* w, void* out, int M, int inter, int K, int pair,
                                      int* error_flag, cudaStream_t stream) {
  if (M <= 0 || inter <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || error_flag == nullptr) return TS_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return TS_ERR_UNSUPPORTED;
  CUtensorMap mx, mw;
  if (!make_map(&mx, x, M, K, TG_BM) || !make_map(&mw, w, 2 * inter, K, 128)) return TS_ERR_UNSUPPORTED;
  if (pair) return launch_tc_pair<6, bf16, true>(mx, mw, (bf16*)out, M, inter, K, error_flag, stream);
  return launch_tc<256, 4, bf16, true>(mx, mw, (bf16*)out, M, inter, K, error_flag, stream);
}
