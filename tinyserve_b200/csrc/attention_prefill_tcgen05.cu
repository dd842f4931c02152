// Varlen causal prefill attention over the paged cache on the 5th-generation tensor cores (bf16,
// head sizes 64 and 128, page sizes 8 or a multiple of 16). Same math as attention_mma.cu
// (upstream src/tinyserve/attention.py:89-111, src/tinyserve/triton_prefill.py:50-125):
// S = Q K^T * scale, causal (and window) mask, softmax in 32-bit, O = P V.
//
// A CTA owns 128 consecutive tokens of one request for NQ query heads of one kv group (NQ = 2
// where the group is even, else 1): the heads share the key and value tiles in shared memory, so
// a tile is fetched once for 256 query rows. Both products run as tcgen05.mma with the
// accumulators in tensor memory:
//   S = Q K^T : A = Q  [128 x D]    K-major, shared memory, 128-byte swizzle
//               B = K  [128 x D]    K-major, the cache rows as TMA delivers them
//   O += P V  : A = P  [128 x 128]  bf16 in tensor memory, written there by the softmax warps over
//                                   the scores they were computed from
//               B = V  [128 x D]    read as it lies in the cache: MN-major (D contiguous)
// Tensor memory, NQ = 1: two score / probability buffers of 128 columns, used by alternate tiles,
// and O; S of tile j + 1 is issued before P V of tile j, so it is computed while the softmax warps
// work on tile j. NQ = 2: one score / probability buffer and O per head (512 columns in all); the
// tensor core alternates between the heads (P V of head 0, S of head 0's next tile, P V of head 1,
// S of head 1's next tile), so it works for one head while the other head's softmax runs.
// Roles:
//   softmax warps : four per head, one thread per row (two heads a CTA), or eight for the one head of a
//               CTA, two threads per row with half of a tile's columns each, which exchange the row
//               maximum through shared memory and meet at a named barrier. A thread reads its part of
//               S (tcgen05.ld), masks, keeps the running maximum and its part of the sum, writes P as
//               bf16 over the first 64 columns of the same buffer (tcgen05.st), and scales O in tensor
//               memory only when the maximum has grown by more than 2^8 (the sum and O then simply carry
//               a common factor that the final division removes); at the end divides O by the sum and
//               stores it
//   TMA warps : K and V tiles of 128 positions (three stages, two for NQ = 2), a box per page part and
//               64 columns, one lane per box; keys and values have warps of their own (one each, or two
//               each for NQ = 1), and the block-table look-up of a tile is made a tile ahead
//   last warp : allocates tensor memory; one lane issues every tcgen05.mma and the
//               tcgen05.commit that tells the other roles what has finished; zeroes V rows
//               outside the live key range (0 x garbage would not be 0). A product that
//               overwrites a buffer is always issued after the product that read P from it, and
//               the tensor core runs them in order.
// Where the time goes (B200, 16 / 8 heads of 128; device clock stamps of one CTA's roles): a tile step
// (128 rows x 128 keys) costs 1,024 cycles of tensor core (16 instructions of 128 x 128 x 16 at the
// measured 64 cycles each) and 1,024 cycles of the exponential unit. With one TMA warp for both
// tensors that warp set the pace: a copy costs its issuing warp about 100 cycles, a tile has 32 of
// them, 3,050 cycles a step; with warps of their own for keys and values the softmax warps set it:
// 2,550 cycles a step with two threads per row (wait for S 210, load 130, maximum 260, exchange 390,
// exponentials and pack 1,240 of which the exponential unit is busy for 1,024, store and hand-over 300):
// 2,048 tokens 41 -> 35 us, 8,192 tokens 640 -> 810 TFLOP/s with one head a CTA. Doing every second
// exponential as a polynomial on the FMA pipe made the step longer (the softmax warps are short of
// issue slots, not only of the exponential unit). With two heads a CTA the tensor core works for one
// head while the other's softmax runs: 920 TFLOP/s at 8,192 tokens. Every operand read from shared
// memory and every TMA write goes through the same 128 bytes per cycle, which is why P stays in tensor
// memory.
// Every wait is on an mbarrier, is bounded and gives up at once when another role has: the CTA
// then records the failure in *error_flag, waits for its copies in flight, frees its tensor
// memory and returns.
#define TS_PDL_CLASS PDL_ATTENTION
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "attention.cuh"
#include "tcgen05.cuh"

namespace ts {

constexpr int FA_BM = 128, FA_BN = 128;
constexpr float FA_RESCALE_STEP = 8.f;      // log2 of the growth of a row maximum that is tolerated without scaling O

__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t fa_pack(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// A wait of a whole warp with one outcome for all its lanes.
__device__ __forceinline__ bool fa_warp_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
  return __all_sync(0xffffffffu, mbar_wait_or_fail(bar, parity, failed) ? 1 : 0) != 0;
}

template <int D64, int NQ>
struct FaLayout {
  static constexpr int D = 64 * D64;
  static constexpr int STAGES = NQ == 1 ? 3 : 2;              // K / V tiles in flight
  static constexpr int SPB = NQ == 1 ? 2 : 1;                 // score / probability buffers per head
  // softmax warps per quarter of the rows, each with BN / HS of a tile's columns: two with one head (the
  // softmax of a tile is the pace there, and two threads per row halve it); with two heads the register
  // file has no room for sixteen softmax warps
  static constexpr int HS = NQ == 1 ? 2 : 1;
  static constexpr int SOFTMAX_WARPS = 4 * HS * NQ;
  static constexpr int PW = NQ == 1 ? 2 : 1;                  // TMA warps per tensor (keys, values)
  static constexpr int THREADS = (SOFTMAX_WARPS + 2 * PW + 1) * 32;      // + the TMA warps and the MMA warp
  static constexpr uint32_t Q_BYTES = FA_BM * D * 2;          // per head
  static constexpr uint32_t KV_BYTES = FA_BN * D * 2;         // one K or V tile
  static constexpr uint32_t OFF_Q = 0;
  static constexpr uint32_t OFF_K = OFF_Q + NQ * Q_BYTES;
  static constexpr uint32_t OFF_V = OFF_K + STAGES * KV_BYTES;
  static constexpr uint32_t TOTAL = OFF_V + STAGES * KV_BYTES;
  // tensor memory columns: the score / probability buffers of every head, then the outputs
  static constexpr uint32_t TMEM_SP = 0, TMEM_O = NQ * SPB * FA_BN;
  static constexpr uint32_t TMEM_COLS = 512;
};

// D64 = head_dim / 64; BR = rows of a tensor box (16, or 8 for pages of 8); NQ = heads per CTA.
// blockIdx = (group of NQ query heads, tile of 128 tokens counted from the end, request in the list).
template <int D64, int BR, int NQ>
__global__ void __launch_bounds__((4 * (NQ == 1 ? 2 : 1) * NQ + 2 * (NQ == 1 ? 2 : 1) + 1) * 32) prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                            const __grid_constant__ CUtensorMap map_v,
                                                                            AttnArgs a, int* error_flag) {
  using L = FaLayout<D64, NQ>;
  constexpr int D = L::D, BN = FA_BN, FA_KV_STAGES = L::STAGES, SPB = L::SPB, FA_SOFTMAX_WARPS = L::SOFTMAX_WARPS, HS = L::HS, PW = L::PW;
  constexpr int HC = BN / HS;                                  // score columns of one softmax thread
  // instruction descriptors: D = f32, A = B = bf16, M = 128; S: N = BN, both operands K-major;
  // PV: N = D, B MN-major (bit 16)
  constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(FA_BM >> 4) << 24);
  constexpr uint32_t IDESC_PV =
      (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(FA_BM >> 4) << 24);
  extern __shared__ unsigned char fa_raw[];
  __shared__ __align__(8) uint64_t k_full[FA_KV_STAGES], k_empty[FA_KV_STAGES], v_full[FA_KV_STAGES], v_empty[FA_KV_STAGES];
  __shared__ __align__(8) uint64_t s_full[NQ][SPB], p_full[NQ][SPB], pv_done[NQ][SPB], q_ready;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed_flag;
  __shared__ float pair_value[NQ][4][HS][32];      // what the warps of a row quarter tell one another: a row maximum, a row sum
  __shared__ int pair_ok[NQ][4][HS];
  volatile int* failed = &failed_flag;

  // ---- which rows and keys (uniform over the CTA); a CTA without rows leaves before any set-up
  const int seq = a.seq_ids[blockIdx.z];
  const int ctx = a.ctx_lens[seq];
  const int q_start = a.cu_q[seq];
  const int q_len = a.cu_q[seq + 1] - q_start;
  const int ntq = (q_len + FA_BM - 1) / FA_BM;
  if ((int)blockIdx.y >= ntq) return;
  const int tile_q = ntq - 1 - (int)blockIdx.y;               // the longest rows first, for every head
  const int q0 = tile_q * FA_BM;
  const int valid = min(FA_BM, q_len - q0);
  const int p_lo = ctx - q_len + q0;                          // position of row 0
  const int p_hi = p_lo + valid - 1;                          // position of the last live row
  const int lo = a.window > 0 ? max(0, p_lo - a.window + 1) : 0;   // first key any row sees
  const int t_begin = lo / BN;
  const int n_tiles = (p_hi + 1 + BN - 1) / BN - t_begin;     // >= 1
  const int head0 = (int)blockIdx.x * NQ;
  const int kvh = head0 / (a.num_heads / a.num_kv_heads);

  pdl_trigger();
  unsigned char* smem = (unsigned char*)(((uintptr_t)fa_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < FA_KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int q = 0; q < NQ; ++q)
      for (int b = 0; b < SPB; ++b) { mbar_init(&s_full[q][b], 1); mbar_init(&p_full[q][b], 4 * HS); mbar_init(&pv_done[q][b], 1); }
    mbar_init(&q_ready, FA_SOFTMAX_WARPS);
    failed_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == FA_SOFTMAX_WARPS + 2 * PW) tmem_alloc(&tmem_base_slot, L::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_wait();      // q and the cache rows of this step are written by the kernels before

  if (warp < FA_SOFTMAX_WARPS) {
    // =========================================================== softmax warps
    // head of this warp, which half of a tile's keys (and of the head's output columns), lane quarter
    const int q = warp / (4 * HS), half = (warp / 4) % HS, quad = warp & 3;
    const int head = head0 + q;
    const int r = quad * 32 + lane;                            // this thread's row
    unsigned char* q_tile = smem + L::OFF_Q + q * L::Q_BYTES;
    {
      // Q rows into the swizzled operand layout: 16 (or 8) threads fetch a row, 16 bytes each
      constexpr int TPH = 128 * HS;                            // softmax threads of a head
      constexpr int CPR = D / 8;                               // 16-byte chunks per row
      constexpr int RPP = TPH / CPR, PASSES = FA_BM / RPP;     // rows per pass of the head's threads
      const int tq = threadIdx.x % TPH;
      const int c = tq % CPR, row0 = tq / CPR;
      uint4 v[PASSES];
#pragma unroll
      for (int i = 0; i < PASSES; ++i) {                       // every load in flight before the first store
        const int row = row0 + i * RPP;
        v[i] = make_uint4(0u, 0u, 0u, 0u);
        if (row < valid)
          v[i] = *reinterpret_cast<const uint4*>((const bf16*)a.q + ((size_t)(q_start + q0 + row) * a.num_heads + head) * D + c * 8);
      }
#pragma unroll
      for (int i = 0; i < PASSES; ++i) {
        const int row = row0 + i * RPP;
        *reinterpret_cast<uint4*>(q_tile + (c >> 3) * (FA_BM * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = v[i];
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_ready);
    }
    // The HS warps of a row quarter meet twice per exchange (named barrier 1 + its index, 32 HS threads):
    // after writing and after reading. Each also says whether its waits have held, so that they stop
    // together: a warp that left alone would leave its partner at the barrier.
    auto pair_sync = [&]() {      // barriers 1 to 4 by literal numbers, so that the assembler counts them
      if (quad == 0) asm volatile("bar.sync 1, 64;" ::: "memory");
      else if (quad == 1) asm volatile("bar.sync 2, 64;" ::: "memory");
      else if (quad == 2) asm volatile("bar.sync 3, 64;" ::: "memory");
      else asm volatile("bar.sync 4, 64;" ::: "memory");
    };
    auto exchange = [&](float mine, bool mine_ok, float (&all)[HS]) -> bool {
      if constexpr (HS == 1) {
        all[0] = mine;
        return mine_ok;
      } else {
        static_assert(HS <= 2 && NQ * (HS - 1) <= 1, "one pair of warps per row quarter, one head");
        pair_value[q][quad][half][lane] = mine;
        if (lane == 0) pair_ok[q][quad][half] = mine_ok ? 1 : 0;
        pair_sync();
        bool all_ok = true;
#pragma unroll
        for (int h2 = 0; h2 < HS; ++h2) {
          all[h2] = pair_value[q][quad][h2][lane];
          all_ok = all_ok && pair_ok[q][quad][h2] != 0;
        }
        pair_sync();
        return all_ok;
      }
    };
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const uint32_t tmem_o = tmem_base + lane_addr + L::TMEM_O + (uint32_t)(q * D);
    const int p_abs = p_lo + r;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true, stopped = false;
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j % SPB, nth = j / SPB;                    // buffer, and how often it has been used
      const uint32_t tmem_sp = tmem_base + lane_addr + L::TMEM_SP + (uint32_t)((q * SPB + b) * BN);
      if (ok && !fa_warp_wait(&s_full[q][b], nth & 1, failed)) ok = false;
      tc_fence_after();
      uint32_t sraw[HC];
      float mx = -INFINITY;
      const int k0 = (t_begin + j) * BN + half * HC;           // the first key of this thread's columns
      if (ok) {
#pragma unroll
        for (int c = 0; c < HC / 32; ++c) tmem_ld_32_nowait(tmem_sp + half * HC + c * 32, sraw + c * 32);
        tmem_ld_wait();
        const bool edge = (k0 + HC - 1 > p_lo) || (a.window > 0 && k0 < p_lo + FA_BM - a.window);
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains: the maxima do not wait on one another
        if (edge) {
          const int first = a.window > 0 ? p_abs - a.window + 1 : 0;
#pragma unroll
          for (int i = 0; i < HC; ++i) {
            const int kpos = k0 + i;
            const float v = (kpos <= p_abs && kpos >= first) ? __uint_as_float(sraw[i]) : -INFINITY;
            sraw[i] = __float_as_uint(v);
            mx4[i & 3] = fmaxf(mx4[i & 3], v);
          }
        } else {
#pragma unroll
          for (int i = 0; i < HC; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sraw[i]));
        }
        mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      }
      // the row's maximum over all its columns; every score of the tile has been read by now, so the
      // probabilities may overwrite them
      float maxima[HS];
      if (!exchange(mx, ok, maxima)) { stopped = true; break; }
#pragma unroll
      for (int h2 = 0; h2 < HS; ++h2) mx = fmaxf(mx, maxima[h2]);
      const float m_new = fmaxf(m_used, mx * a.scale_log2);
      if (j == 0) {
        m_used = m_new;
      } else {
        const bool grow = m_new > m_used + FA_RESCALE_STEP;    // also when nothing was seen before (-inf)
        if (__any_sync(0xffffffffu, grow)) {
          // O is final up to tile j - 1 before it is scaled; each warp scales its share of the columns
          if (!fa_warp_wait(&pv_done[q][(j - 1) % SPB], ((j - 1) / SPB) & 1, failed)) ok = false;
          tc_fence_after();
          const float alpha = grow ? (m_used == -INFINITY ? 0.f : fa_exp2(m_used - m_new)) : 1.f;
          if (ok) {
#pragma unroll 1
            for (int c = half * (D / 32 / HS); c < (half + 1) * (D / 32 / HS); ++c) {
              uint32_t o[32];
              tmem_ld_32(tmem_o + c * 32, o);
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st_32(tmem_o + c * 32, o);
            }
          }
          if (grow) { l_sum *= alpha; m_used = m_new; }
        }
      }
      const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
      float add4[4] = {0.f, 0.f, 0.f, 0.f};
      // P as bf16, two keys per 32-bit column, over the first half of this buffer's columns
#pragma unroll
      for (int c = 0; c < HC / 64; ++c) {
        uint32_t packed[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float p0 = fa_exp2(fmaf(__uint_as_float(sraw[c * 64 + 2 * i]), a.scale_log2, -m_sub));
          const float p1 = fa_exp2(fmaf(__uint_as_float(sraw[c * 64 + 2 * i + 1]), a.scale_log2, -m_sub));
          add4[i & 3] += p0 + p1;
          packed[i] = fa_pack(p0, p1);
        }
        tmem_st_32_nowait(tmem_sp + half * (HC / 2) + c * 32, packed);
      }
      l_sum += (add4[0] + add4[1]) + (add4[2] + add4[3]);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[q][b]);
    }
    if (!stopped) {
      const int last = n_tiles - 1;
      if (ok && !fa_warp_wait(&pv_done[q][last % SPB], (last / SPB) & 1, failed)) ok = false;
      float sums[HS];
      ok = exchange(l_sum, ok, sums);
      l_sum = 0.f;
#pragma unroll
      for (int h2 = 0; h2 < HS; ++h2) l_sum += sums[h2];      // in the order of the columns, the same in every warp
    }
    if (ok && !stopped) {
      tc_fence_after();
      const float inv = 1.f / l_sum;
      bf16* dst = (bf16*)a.out + ((size_t)(q_start + q0 + r) * a.num_heads + head) * D;
#pragma unroll 1
      for (int c = half * (D / 32 / HS); c < (half + 1) * (D / 32 / HS); ++c) {
        uint32_t o[32];
        tmem_ld_32(tmem_o + c * 32, o);
        if (r < valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            v.x = fa_pack(__uint_as_float(o[i + 0]) * inv, __uint_as_float(o[i + 1]) * inv);
            v.y = fa_pack(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            v.z = fa_pack(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            v.w = fa_pack(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
          }
        }
      }
    }
  } else if (warp < FA_SOFTMAX_WARPS + 2 * PW) {
    // =========================================================== TMA producers: PW warps for the keys, PW for the values
    // (a copy costs its issuing warp about 100 cycles, a tile has 16 to 32 of them per tensor: one warp
    // for both tensors needed 3,000 cycles a tile and was the slowest role of the CTA). The warps of a
    // tensor take alternate copies of a tile; the first of them arms the tile's barrier (a copy of the
    // other warp that lands before that only makes the byte count negative for a while: the phase
    // cannot end before the arming thread has arrived).
    const int which = (warp - FA_SOFTMAX_WARPS) % 2;            // 0: keys, 1: values
    const int pw = (warp - FA_SOFTMAX_WARPS) / 2;               // which of the tensor's warps
    const int* table = a.block_tables + (size_t)seq * a.table_width;
    constexpr int PARTS = BN / BR;
    constexpr int COPIES = PARTS * D64;                         // per tile and tensor: one lane each
    static_assert(COPIES <= 32, "a lane issues at most one copy per tile and tensor");
    const int kmin = lo & ~(BR - 1), kmax = (ctx - 1) & ~(BR - 1);
    const int copy = lane * PW + pw;                            // this lane's copy of a tile
    const int part = copy / D64, h = copy - part * D64;         // its part of the tile and half of the head
    // The row of the cache tensors where this lane's part of tile j begins: a look-up in the block
    // table, the same for keys and values. It is fetched a tile ahead: looked up when the copies
    // are due (twice per tile, a trip to L2 each time) it made this warp the slowest role of the CTA
    // (3,000 cycles a tile against 1,024 of tensor core and 2,100 of softmax).
    auto cache_row = [&](int j) -> int {
      // a part wholly outside the live keys is fetched from the nearest live part (its scores are
      // masked and its value rows zeroed); every part lies within one page
      const int kpos = min(max((t_begin + j) * BN + part * BR, kmin), kmax);
      int page, off;
      if (a.page_shift >= 0) { page = table[kpos >> a.page_shift]; off = kpos & (a.page_size - 1); }
      else { const int idx = kpos / a.page_size; page = table[idx]; off = kpos - idx * a.page_size; }
      return (page * a.num_kv_heads + kvh) * a.page_size + off;
    };
    bool ok = !wait_test_unarmed();
    int issued = 0;
    uint64_t* const full_bars = which == 0 ? k_full : v_full;
    uint64_t* const empty_bars = which == 0 ? k_empty : v_empty;
    const CUtensorMap* const map = which == 0 ? &map_k : &map_v;
    const bool mine = copy < COPIES;
    int y = mine ? cache_row(0) : 0;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j % FA_KV_STAGES;
      const uint32_t ph = (j / FA_KV_STAGES) & 1;
      const int y_next = (mine && j + 1 < n_tiles) ? cache_row(j + 1) : 0;      // in flight during this tile's wait
      int good = 1;
      if (lane == 0) {
        good = mbar_wait_or_fail(&empty_bars[st], ph ^ 1, failed) ? 1 : 0;
        if (good && pw == 0) mbar_expect_tx(&full_bars[st], L::KV_BYTES);
      }
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { ok = false; break; }
      unsigned char* dst = smem + (which == 0 ? L::OFF_K : L::OFF_V) + st * L::KV_BYTES;
      if (mine) tma_load_2d(dst + h * (BN * 128) + part * (BR * 128), map, &full_bars[st], h * 64, y);
      issued = j + 1;
      y = y_next;
    }
    if (!ok && lane == 0) {
      // leave no copy in flight: the last phases armed on every stage must complete
      for (int back = 0; back < FA_KV_STAGES; ++back) {
        const int jj = issued - 1 - back;
        if (jj >= 0) mbar_wait(&full_bars[jj % FA_KV_STAGES], (jj / FA_KV_STAGES) & 1);
      }
    }
  } else {
    // =========================================================== MMA issuer
    bool ok = fa_warp_wait(&q_ready, 0, failed);
    const uint32_t q_addr = smem_u32(smem + L::OFF_Q);
    const uint32_t k_addr = smem_u32(smem + L::OFF_K), v_addr = smem_u32(smem + L::OFF_V);
    // S_q = Q_q K^T of tile j into the head's buffer j % SPB
    auto issue_s = [&](int j, int q) {
      const int st = j % FA_KV_STAGES, bq = q * SPB + j % SPB;
      if (lane == 0) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint64_t ad = sw128_desc(q_addr + q * L::Q_BYTES + (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32);
          const uint64_t bd = sw128_desc(k_addr + st * L::KV_BYTES + (ks >> 2) * (BN * 128) + (ks & 3) * 32);
          umma_bf16(tmem_base + L::TMEM_SP + (uint32_t)(bq * BN), ad, bd, IDESC_S, ks != 0);
        }
        umma_commit(&s_full[q][j % SPB]);
        if (q == NQ - 1) umma_commit(&k_empty[st]);       // the K stage is free once the last head's S has read it
      }
      __syncwarp();
    };
    // O_q += P_q V of tile j, P read from the head's buffer in tensor memory
    auto issue_pv = [&](int j, int q) -> bool {
      const int st = j % FA_KV_STAGES, b = j % SPB;
      if (!fa_warp_wait(&p_full[q][b], (j / SPB) & 1, failed)) return false;
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          const uint64_t bd = sw128_desc_mn(v_addr + st * L::KV_BYTES + ks * (16 * 128), BN * 128);
          umma_bf16_ta(tmem_base + L::TMEM_O + (uint32_t)(q * D),
                       tmem_base + L::TMEM_SP + (uint32_t)((q * SPB + b) * BN + ks * 8), bd, IDESC_PV, (j | ks) != 0);
        }
        umma_commit(&pv_done[q][b]);
        if (q == NQ - 1) umma_commit(&v_empty[st]);
      }
      __syncwarp();
      return true;
    };
    auto k_ready = [&](int j) -> bool {
      const bool got = fa_warp_wait(&k_full[j % FA_KV_STAGES], (j / FA_KV_STAGES) & 1, failed);
      tc_fence_after();
      return got;
    };
    // V of tile j is there; its rows of positions outside [lo, ctx) may hold anything: zero them (their P is 0)
    auto v_ready = [&](int j) -> bool {
      const int st = j % FA_KV_STAGES;
      if (!fa_warp_wait(&v_full[st], (j / FA_KV_STAGES) & 1, failed)) return false;
      const int k0 = (t_begin + j) * BN;
      if (k0 < lo || k0 + BN > ctx) {
        unsigned char* v_tile = smem + L::OFF_V + st * L::KV_BYTES;
        for (int idx = lane; idx < BN * D64 * 8; idx += 32) {
          const int row = idx / (D64 * 8), c = idx - row * (D64 * 8);
          const int kpos = k0 + row;
          if (kpos < lo || kpos >= ctx)
            *reinterpret_cast<uint4*>(v_tile + (c >> 3) * (BN * 128) + row * 128 + ((c & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async_smem();
        __syncwarp();
      }
      return true;
    };
    if (ok) ok = k_ready(0);
    if (ok) {
      for (int q = 0; q < NQ; ++q) issue_s(0, q);
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      const bool more = j + 1 < n_tiles;
      if constexpr (NQ == 1) {
        // two buffers: the next tile's scores are computed while the softmax warps work on this one
        if (more) {
          ok = k_ready(j + 1);
          if (!ok) break;
          issue_s(j + 1, 0);
        }
        ok = v_ready(j) && issue_pv(j, 0);
      } else {
        // one buffer per head: a head's next scores follow the product that read its P; meanwhile
        // the other head's softmax runs
        ok = v_ready(j);
        if (ok && more) ok = k_ready(j + 1);
        for (int q = 0; q < NQ && ok; ++q) {
          ok = issue_pv(j, q);
          if (ok && more) issue_s(j + 1, q);
        }
      }
    }
  }
  if (*failed && (threadIdx.x & 31) == 0) atomicExch(error_flag, WAIT_FAILED_PREFILL_TCGEN05);
  tc_fence_before();
  __syncthreads();
  if (warp == FA_SOFTMAX_WARPS + 2 * PW) tmem_dealloc(tmem_base, L::TMEM_COLS);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*FaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The descriptor of one cache tensor ([rows, head_dim] bf16, boxes of box_rows x 64, 128-byte
// swizzle), kept per (address, rows, head_dim, box_rows): a cache tensor is allocated once.
static const CUtensorMap* fa_cache_map(const void* base, long long rows, int head_dim, int box_rows) {
  static std::mutex mu;
  static std::map<std::tuple<const void*, long long, int, int>, CUtensorMap> maps;
  static FaEncodeFn fn = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_tuple(base, rows, head_dim, box_rows);
  auto it = maps.find(key);
  if (it != maps.end()) return &it->second;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = (FaEncodeFn)p;
  }
  CUtensorMap m;
  cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return nullptr;
  return &maps.emplace(key, m).first->second;
}

template <int D64, int BR, int NQ>
static int launch_fa(const AttnArgs& a, long long cache_rows, int max_query_len, int* error_flag, cudaStream_t stream) {
  using L = FaLayout<D64, NQ>;
  const CUtensorMap* mk = fa_cache_map(a.k_cache, cache_rows, L::D, BR);
  const CUtensorMap* mv = fa_cache_map(a.v_cache, cache_rows, L::D, BR);
  if (mk == nullptr || mv == nullptr) return TS_ERR_UNSUPPORTED;
  const size_t smem = (size_t)L::TOTAL + 1024;
  auto kern = prefill_attn_tc_kernel<D64, BR, NQ>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(a.num_heads / NQ, (max_query_len + FA_BM - 1) / FA_BM, a.num_seqs);
  return launch(kern, grid, L::THREADS, smem, stream, *mk, *mv, a, error_flag);
}

}  // namespace ts

using namespace ts;

// bf16 prefill attention on tcgen05 for the requests listed in prefill_seqs. head_dim 64 or 128;
// page_size 8 or a multiple of 16; num_pages_total = pages of the cache tensors (the pad page
// included). heads_per_cta: 1, or 2 query heads of a kv group sharing a CTA's key and value tiles
// (needs an even group); 0 picks 2 where it can. Returns TS_ERR_UNSUPPORTED for sizes it does
// not take.
extern "C" int ts_prefill_attention_tcgen05(
    const void* q, void* out, const void* k_cache, const void* v_cache, long long num_pages_total,
    const int* block_tables, int table_width, const int* cu_q, const int* ctx_lens, const int* prefill_seqs,
    int num_prefill, int max_query_len, int num_heads, int num_kv_heads, int head_dim, int page_size, float scale,
    int window, int heads_per_cta, int* error_flag, cudaStream_t stream) {
  if (num_prefill <= 0 || max_query_len <= 0) return 0;
  if ((head_dim != 64 && head_dim != 128) || error_flag == nullptr) return TS_ERR_UNSUPPORTED;
  if (!(page_size == 8 || (page_size > 0 && page_size % 16 == 0))) return TS_ERR_UNSUPPORTED;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || window < 0 || num_pages_total <= 0) return TS_ERR_BAD_ARGUMENT;
  if ((((uintptr_t)k_cache) | ((uintptr_t)v_cache) | ((uintptr_t)q) | ((uintptr_t)out)) & 15) return TS_ERR_UNSUPPORTED;
  const long long rows = num_pages_total * num_kv_heads * page_size;
  if (rows >= (1ll << 31)) return TS_ERR_UNSUPPORTED;
  const int group = num_heads / num_kv_heads;
  if (heads_per_cta == 0) heads_per_cta = (group % 2 == 0) ? 2 : 1;
  if (heads_per_cta != 1 && heads_per_cta != 2) return TS_ERR_BAD_ARGUMENT;
  if (heads_per_cta == 2 && group % 2 != 0) return TS_ERR_UNSUPPORTED;
  AttnArgs a;
  a.q = q; a.out = out; a.k_cache = k_cache; a.v_cache = v_cache;
  a.block_tables = block_tables; a.table_width = table_width; a.cu_q = cu_q; a.ctx_lens = ctx_lens;
  a.seq_ids = prefill_seqs; a.num_seqs = num_prefill;
  a.num_heads = num_heads; a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.page_size = page_size;
  a.page_shift = page_shift_of(page_size);
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  a.num_splits = 1; a.part_acc = nullptr; a.part_ml = nullptr;
#define TS_FA(D64_, BR_)                                                                                \
  return heads_per_cta == 2 ? launch_fa<D64_, BR_, 2>(a, rows, max_query_len, error_flag, stream)       \
                            : launch_fa<D64_, BR_, 1>(a, rows, max_query_len, error_flag, stream)
  if (head_dim == 64) {
    if (page_size == 8) { TS_FA(1, 8); }
    TS_FA(1, 16);
  }
  if (page_size == 8) { TS_FA(2, 8); }
  TS_FA(2, 16);
#undef TS_FA
}
