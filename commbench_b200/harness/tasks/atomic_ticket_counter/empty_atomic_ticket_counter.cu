// A ticket counter hammered by several independent producers: every producer (one kernel of one
// thread on its own stream, standing for one processing element of a partitioned-global-address
// program) performs `ops` system-scope fetch-and-increment operations on ONE 64-bit counter and
// records the tickets it drew.  Over all producers every ticket 0 .. P*ops-1 must appear exactly
// once.  The kernels never wait for each other, so running them as separate launches on one GPU
// is safe.  Reports the cost per atomic from the device's cycle counter.  Prints one JSON object.
#include <cuda_runtime.h>

#include <algorithm>
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

constexpr int kProducers = 4;

// One thread.  tickets[i] = value the counter held before this producer's i-th increment;
// *cycles = clock64() ticks spent in the loop.
__global__ void ticket_kernel(unsigned long long* counter, int ops, unsigned long long* tickets,
                              unsigned long long* cycles) {
  // TODO: one thread; time the loop of `ops` atomicAdd_system(counter, 1ull) calls with
  //       clock64() and store every returned ticket
}

int main() {
  const int sweeps[] = {1, 16, 256, 4096, 10240};
  const int max_ops = 10240;
  unsigned long long *counter = nullptr, *tickets = nullptr, *cycles = nullptr;
  CK(cudaMalloc(&counter, sizeof(unsigned long long)));
  CK(cudaMalloc(&tickets, sizeof(unsigned long long) * kProducers * max_ops));
  CK(cudaMalloc(&cycles, sizeof(unsigned long long) * kProducers));
  cudaStream_t streams[kProducers];
  for (int p = 0; p < kProducers; ++p) CK(cudaStreamCreateWithFlags(&streams[p], cudaStreamNonBlocking));
  int khz = 0;
  CK(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, 0));
  bool ok = true;
  std::vector<double> cycles_per_op;
  std::vector<unsigned long long> host(static_cast<size_t>(kProducers) * max_ops), hc(kProducers);
  for (int ops : sweeps) {
    CK(cudaMemset(counter, 0, sizeof(unsigned long long)));
    CK(cudaMemset(tickets, 0xff, sizeof(unsigned long long) * kProducers * max_ops));
    CK(cudaMemset(cycles, 0, sizeof(unsigned long long) * kProducers));
    CK(cudaDeviceSynchronize());
    for (int p = 0; p < kProducers; ++p)
      ticket_kernel<<<1, 32, 0, streams[p]>>>(counter, ops, tickets + static_cast<size_t>(p) * max_ops, cycles + p);
    CK(cudaGetLastError());
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(host.data(), tickets, sizeof(unsigned long long) * kProducers * max_ops, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(hc.data(), cycles, sizeof(unsigned long long) * kProducers, cudaMemcpyDeviceToHost));
    unsigned long long final_value = 0;
    CK(cudaMemcpy(&final_value, counter, sizeof(final_value), cudaMemcpyDeviceToHost));
    std::vector<unsigned long long> all;
    for (int p = 0; p < kProducers; ++p) {
      const unsigned long long* mine = host.data() + static_cast<size_t>(p) * max_ops;
      for (int i = 0; i < ops; ++i) {
        all.push_back(mine[i]);
        if (i > 0) ok = ok && mine[i] > mine[i - 1];   // one producer's tickets only grow
      }
      ok = ok && hc[p] > 0;
    }
    std::sort(all.begin(), all.end());
    ok = ok && final_value == static_cast<unsigned long long>(kProducers) * ops;
    for (size_t i = 0; i < all.size(); ++i) ok = ok && all[i] == i;      // each ticket exactly once
    double worst = 0;
    for (int p = 0; p < kProducers; ++p) worst = std::max(worst, static_cast<double>(hc[p]) / ops);
    cycles_per_op.push_back(worst);
  }
  printf("{\"Correctness\": \"%s\", \"producers\": %d, \"data_size_unit\": \"ops per producer\", "
         "\"latency_unit\": \"us\", \"throughput_unit\": \"Mops/s\", \"metrics\": [",
         ok ? "PASS" : "FAIL", kProducers);
  for (size_t i = 0; i < cycles_per_op.size(); ++i) {
    const double us = cycles_per_op[i] / (khz / 1e3);
    printf("%s{\"data_size\": %d, \"cycles_per_op\": %.1f, \"latency_avg\": %.4f, \"throughput_avg\": %.3f}",
           i ? ", " : "", sweeps[i], cycles_per_op[i], us, us > 0 ? kProducers / us : 0.0);
  }
  printf("]}\n");
  return ok ? 0 : 1;
}
