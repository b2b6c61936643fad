// Shared-memory mbarrier wrappers with bounded waits.
//
// Same instruction set as the producer/consumer microbenchmark of
// datasets/example072_GPU_barrier_within_CTA/nv/empty_gpu_barrier_within_cta.cu:44-65
// (init / arrive / try_wait.parity), plus expect_tx for TMA completion
// (datasets/example094_TMA_bulk_copy_gmem_to_smem/nv/empty_tma_bulk_copy.cu:28-58).
#pragma once
#include "ptx.cuh"

namespace cb {

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)
               : "memory");
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Makes mbarrier.init visible to the async proxy (TMA, tcgen05.commit).
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_addr(uint32_t bar_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_addr),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait.  `abort_flag` is a CTA-shared word: once any role of the CTA
// gives up, every other waiting role leaves too, so the CTA can reach its
// tear-down (drain copies, free TMEM) instead of deadlocking on itself.
// Two limits: a poll count and a %globaltimer budget of 4 s, whichever comes
// first; both are far above any legitimate wait here.
#define CB_MBAR_SPIN_LIMIT (1u << 28)
#define CB_MBAR_TIMEOUT_NS 4000000000ull

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t* status, uint32_t detail) {
  uint64_t t0 = 0;
  for (uint32_t it = 0; it < CB_MBAR_SPIN_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u) {
      if (abort_flag != nullptr && *abort_flag != 0) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > CB_MBAR_TIMEOUT_NS) break;
    }
  }
  if (abort_flag != nullptr) *abort_flag = 1;
  report_status(status, CB_TIMEOUT_MBARRIER, 0, detail);
  return false;
}

}  // namespace cb
