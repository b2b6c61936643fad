// Device-side time: read %globaltimer, measure how long __nanosleep(n) really sleeps for
// n = 100 ns .. 1 ms, and find the timer's resolution.  Prints one JSON object.
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

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  // TODO: read the %globaltimer special register (nanoseconds)
  return 0;
}

// out[0] = mean slept ns over `reps`, out[1] = smallest observed ns, out[2] = largest.
__global__ void sleep_probe_kernel(unsigned request_ns, int reps, unsigned long long* out) {
  // TODO: one thread; per repetition read the timer, __nanosleep(request_ns), read it again.
}

// out[0] = smallest non-zero step between consecutive reads; out[1] = 1 if the timer never ran backwards.
__global__ void resolution_kernel(unsigned long long* out) {
  // TODO: one thread, 65536 back-to-back reads.
}

int main() {
  const unsigned requests[] = {100, 1000, 10000, 100000, 1000000};
  unsigned long long* d = nullptr;
  CK(cudaMalloc(&d, 4 * sizeof(unsigned long long)));
  CK(cudaMemset(d, 0, 4 * sizeof(unsigned long long)));
  bool ok = true;
  unsigned long long h[4] = {0, 0, 0, 0};
  resolution_kernel<<<1, 32>>>(d);
  CK(cudaDeviceSynchronize());
  CK(cudaMemcpy(h, d, 2 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
  const unsigned long long resolution = h[0];
  ok = ok && h[1] == 1 && resolution > 0 && resolution <= 1000000ull;
  std::vector<double> mean, lo, hi;
  for (unsigned r : requests) {
    sleep_probe_kernel<<<1, 32>>>(r, 50, d);
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(h, d, 3 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    mean.push_back(static_cast<double>(h[0]));
    lo.push_back(static_cast<double>(h[1]));
    hi.push_back(static_cast<double>(h[2]));
    // The hardware may sleep anywhere in [0, 2 * request]; with the timer's granularity on top.
    ok = ok && h[0] > 0 && static_cast<double>(h[0]) <= 2.0 * r + 2.0 * resolution + 20000.0;
  }
  // CUDA events and the device timer must agree on a ~20 ms interval within 20 %
  sleep_probe_kernel<<<1, 32>>>(0, 1, d);
  CK(cudaDeviceSynchronize());
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  CK(cudaEventRecord(e0));
  sleep_probe_kernel<<<1, 32>>>(1000000, 20, d);
  CK(cudaEventRecord(e1));
  CK(cudaEventSynchronize(e1));
  float ms = 0.f;
  CK(cudaEventElapsedTime(&ms, e0, e1));
  CK(cudaMemcpy(h, d, 3 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
  const double device_ms = static_cast<double>(h[0]) * 20 / 1e6;
  ok = ok && device_ms > 0 && ms > 0 && device_ms / ms > 0.8 && device_ms / ms < 1.2;
  printf("{\"Correctness\": \"%s\", \"timer_resolution_ns\": %llu, \"event_ms\": %.3f, \"device_ms\": %.3f, "
         "\"data_size_unit\": \"ns requested\", \"latency_unit\": \"us\", \"throughput_unit\": \"ratio\", "
         "\"metrics\": [", ok ? "PASS" : "FAIL", resolution, ms, device_ms);
  for (size_t i = 0; i < mean.size(); ++i)
    printf("%s{\"data_size\": %u, \"latency_avg\": %.3f, \"latency_min\": %.3f, \"latency_max\": %.3f, "
           "\"throughput_avg\": %.3f}",
           i ? ", " : "", requests[i], mean[i] / 1e3, lo[i] / 1e3, hi[i] / 1e3, mean[i] / requests[i]);
  printf("]}\n");
  return ok ? 0 : 1;
}
