// Bounded waits of the kernels that wait on mbarriers (TMA copies, tcgen05 commits): how long a wait
// may last, and what a kernel does when it runs out.
//
// A wait spins until the barrier's phase completes or `wait_cycles()` clock cycles have passed
// (default about a second, far beyond any real wait). A kernel whose wait ran out stops waiting,
// stores its code (WAIT_FAILED_* below) in the error word the launcher was given, frees what it
// holds (tensor memory) and returns; the host reads the word with the step's sampled tokens and
// raises. Nothing ever spins without a bound.
//
// Both knobs live in constant memory, one copy per translation unit (the library is linked without
// relocatable device code), set for all of them by ts_set_wait_control(cycles, unarmed):
//   cycles   the bound in clock cycles;
//   unarmed  test switch: the copy-issuing thread of every kernel skips its copies AND the
//            expect-tx that arms the barrier for them, exactly as if the copies had been lost, so
//            that the consumers' waits run out. With a bound of a few thousand cycles this shows
//            on a healthy GPU, in microseconds, that a lost copy ends as an error code and not as
//            a hang. Never set outside tests.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ts {

constexpr int WAIT_FAILED_GEMM_TCGEN05 = 1, WAIT_FAILED_PREFILL_TCGEN05 = 2, WAIT_FAILED_PREFILL_TMA = 3,
              WAIT_FAILED_DECODE_TMA = 4, WAIT_FAILED_DECODE_BULK = 5;

static __constant__ long long c_wait_cycles = 2000000000ll;
static __constant__ int c_wait_unarmed = 0;

__device__ __forceinline__ long long wait_cycles() { return c_wait_cycles; }
__device__ __forceinline__ bool wait_test_unarmed() { return c_wait_unarmed != 0; }

// mbarrier.try_wait on shared-memory address `addr` for the phase of `parity`; false if the bound was hit.
__device__ __forceinline__ bool bounded_mbar_wait(uint32_t addr, uint32_t parity) {
  const long long start = clock64();
  const long long limit = wait_cycles();
  for (uint32_t i = 0;; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 63u) == 63u && clock64() - start > limit) return false;
  }
}

typedef int (*WaitControlSetter)(long long, int);
extern "C" void ts_wait_control_register(WaitControlSetter setter);   // wait_control.cu

static int wait_control_set(long long cycles, int unarmed) {
  cudaError_t e = cudaMemcpyToSymbol(c_wait_cycles, &cycles, sizeof(cycles));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(c_wait_unarmed, &unarmed, sizeof(unarmed));
  return (int)e;
}
static const int wait_control_registered = (ts_wait_control_register(&wait_control_set), 0);

}  // namespace ts
