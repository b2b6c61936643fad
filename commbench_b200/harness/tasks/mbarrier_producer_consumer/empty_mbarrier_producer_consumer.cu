// Producer/consumer hand-off inside one CTA through two shared-memory mbarriers: thread 0
// publishes a value and arrives on `ready`; every thread of the other warps waits on `ready`
// (try_wait.parity), checks the value and arrives on `consumed`; thread 0 waits on `consumed`
// before the next round.  Reports cycles per round for several CTA sizes.  Prints one JSON object.
//
// Every wait must be bounded: a wait that runs out sets a bit in `errors` and the kernel returns.
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
  // TODO: mbarrier.init.shared::cta.b64
}
__device__ __forceinline__ void mbarrier_arrive(uint64_t* bar) {
  // TODO: mbarrier.arrive.shared::cta.b64 (discard the state)
}
__device__ __forceinline__ bool mbarrier_try_wait(uint64_t* bar, uint32_t parity) {
  // TODO: mbarrier.try_wait.parity.shared::cta.b64 -> true when the phase with this parity is over
  return false;
}
// At most `limit` polls; false when the phase did not complete.
__device__ __forceinline__ bool mbarrier_wait(uint64_t* bar, uint32_t parity, uint32_t limit = 1u << 24) {
  // TODO
  return false;
}

// blockDim.x >= 64: warp 0 holds the producer (lane 0), warps 1.. are consumers.
__global__ void handoff_kernel(int rounds, unsigned long long* cycles, uint32_t* errors) {
  // TODO:
  //  * two mbarriers in shared memory: `ready` (1 arrival) and `consumed` (blockDim.x - 32 arrivals),
  //    initialised by one thread, made visible (fence.mbarrier_init), then __syncthreads();
  //  * per round r: thread 0 writes value = 0x1000 + r to shared memory, arrives on `ready`, waits
  //    on `consumed`; threads >= 32 wait on `ready`, check the value (bit 2 of *errors on a
  //    mismatch), arrive on `consumed`;
  //  * a wait that runs out sets bit 0 (producer) or bit 1 (consumer) of *errors and makes every
  //    thread leave the loop;
  //  * thread 0 stores the clock64() cycles of the whole loop to *cycles.
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
    CK(cudaMemset(d_cycles, 0, sizeof(unsigned long long)));
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
           i ? ", " : "", sizes[i], per_round_cycles[i], us, us > 0 ? 1.0 / us : 0.0);
  }
  printf("]}\n");
  return ok ? 0 : 1;
}
