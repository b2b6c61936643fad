// Device-to-device copy bandwidth with a hand-written kernel.  Prints one JSON object.
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

__global__ void copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t nvec) {
  // TODO: grid-stride loop moving one 16-byte vector per thread and iteration.
}

int main() {
  const size_t sizes[] = {1ull << 20, 16ull << 20, 256ull << 20, 1ull << 30};
  std::vector<double> gbs, us;
  bool ok = true;
  for (size_t nbytes : sizes) {
    uint8_t *src = nullptr, *dst = nullptr;
    CK(cudaMalloc(&src, nbytes));
    CK(cudaMalloc(&dst, nbytes));
    CK(cudaMemset(src, 0x5a, nbytes));
    CK(cudaMemset(dst, 0, nbytes));
    // TODO: pick a launch shape (a multiple of the SM count), run 3 warm-up and 10 timed
    // launches between two CUDA events, store microseconds per launch in `us` and
    // (2 * nbytes) / time in GB/s in `gbs`.
    // TODO: copy the first and last 4 KB of dst back and compare every byte with 0x5a
    // (clear `ok` on a mismatch).
    CK(cudaFree(src));
    CK(cudaFree(dst));
  }
  ok = ok && gbs.size() == sizeof(sizes) / sizeof(sizes[0]);  // nothing measured is not a pass
  printf("{\"Correctness\": \"%s\", \"data_size_unit\": \"MB\", \"latency_unit\": \"us\", "
         "\"throughput_unit\": \"GB/s\", \"metrics\": [", ok ? "PASS" : "FAIL");
  for (size_t i = 0; i < gbs.size(); ++i)
    printf("%s{\"data_size\": %zu, \"latency_avg\": %.3f, \"throughput_avg\": %.3f}", i ? ", " : "",
           sizes[i] >> 20, us[i], gbs[i]);
  printf("]}\n");
  return ok ? 0 : 1;
}
