// Producer/consumer hand-off inside one CTA through two shared-memory mbarriers: thread 0
// publishes a value and arrives on `ready`; every thread of the other warps waits on `ready`
// (try_wait.parity), checks the value and arrives on `consumed`; thread 0 waits on `consumed`
// before the next round.  Reports cycles per round for several CTA sizes.  Prints one JSON object.
//
// Same exercise as the reference's datasets/example072_GPU_barrier_within_CTA (wrappers :44-65,
// benchmark kernel :69-84, block sizes 32..256 and 4096 rounds :236).  Every wait is bounded: a
// wait that runs out sets an error word and the kernel returns.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <vector>

#define CK(x)                                                                       \
  do {                                                                              \
    cudaError_t e_ = (x);                                                           \
    if (e_ != cudaSuccess) {                                                        \
      printf("{\"Correctness\": \"FAIL\", \"error\": \"%s\"}\n", cudaGetErrorString(e_)); \
      return 1;                                                                     \
    }                                                                               \
  } while (0)

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbarrier_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarrier_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbarrier_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// At most `limit` polls; false when the phase did not complete.
__device__ __forceinline__ bool mbarrier_wait(uint64_t* bar, uint32_t parity, uint32_t limit = 1u << 24) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbarrier_try_wait(bar, parity)) return true;
  return false;
}

// blockDim.x >= 64: warp 0 holds the producer (lane 0), warps 1.. are consumers.
__global__ void handoff_kernel(int rounds, unsigned long long* cycles, uint32_t* errors) {
  __shared__ uint64_t ready, consumed;
  __shared__ volatile uint32_t value;
  __shared__ volatile int give_up;
  const uint32_t consumers = blockDim.x - 32;
  if (threadIdx.x == 0) {
    mbarrier_init(&ready, 1);
    mbarrier_init(&consumed, consumers);
    value = 0;
    give_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const long long t0 = clock64();
  for (int r = 0; r < rounds; ++r) {
    const uint32_t parity = static_cast<uint32_t>(r) & 1u;
    if (give_up) break;
    if (threadIdx.x == 0) {
      value = 0x1000u + r;
      mbarrier_arrive(&ready);  // arrive has release semantics: the value is visible to waiters
      if (!mbarrier_wait(&consumed, parity)) {
        atomicOr(errors, 1u);
        give_up = 1;
      }
    } else if (threadIdx.x >= 32) {
      if (!mbarrier_wait(&ready, parity)) {
        atomicOr(errors, 2u);
        give_up = 1;
        break;
      }
      if (value != 0x1000u + r) atomicOr(errors, 4u);
      mbarrier_arrive(&consumed);
    }
  }
  if (threadIdx.x == 0) *cycles = static_cast<unsigned long long>(clock64() - t0);
}

int main() {
  const int sizes[] = {64, 128, 256, 512};
  const int rounds = 4096;
  unsigned long long* d_cycles = nullptr;
  uint32_t* d_err = nullptr;
  CK(cudaMalloc(&d_cycles, sizeof(unsigned long long)));
  CK(cudaMalloc(&d_err, sizeof(uint32_t)));
  int khz = 0;
  CK(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, 0));
  bool ok = true;
  std::vector<double> per_round_cycles;
  for (int threads : sizes) {
    CK(cudaMemset(d_err, 0, sizeof(uint32_t)));
    handoff_kernel<<<1, threads>>>(16, d_cycles, d_err);  // warm-up
    handoff_kernel<<<1, threads>>>(rounds, d_cycles, d_err);
    CK(cudaDeviceSynchronize());
    unsigned long long cyc = 0;
    uint32_t err = 0;
    CK(cudaMemcpy(&cyc, d_cycles, sizeof(cyc), cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(&err, d_err, sizeof(err), cudaMemcpyDeviceToHost));
    ok = ok && err == 0 && cyc > 0;
    per_round_cycles.push_back(static_cast<double>(cyc) / rounds);
  }
  printf("{\"Correctness\": \"%s\", \"data_size_unit\": \"threads\", \"latency_unit\": \"us\", "
         "\"throughput_unit\": \"Mrounds/s\", \"metrics\": [", ok ? "PASS" : "FAIL");
  for (size_t i = 0; i < per_round_cycles.size(); ++i) {
    const double us = per_round_cycles[i] / (khz / 1e3);
    printf("%s{\"data_size\": %d, \"cycles_per_round\": %.1f, \"latency_avg\": %.4f, \"throughput_avg\": %.3f}",
           i ? ", " : "", sizes[i], per_round_cycles[i], us, 1.0 / us);
  }
  printf("]}\n");
  return ok ? 0 : 1;
}
