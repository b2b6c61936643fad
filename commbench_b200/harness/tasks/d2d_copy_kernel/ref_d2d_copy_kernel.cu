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
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  // Four independent loads in flight per thread before the first store.
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a;
    dst[i + stride] = b;
    dst[i + 2 * stride] = c;
    dst[i + 3 * stride] = d;
  }
  for (; i < nvec; i += stride) dst[i] = src[i];
}

int main() {
  const size_t sizes[] = {1ull << 20, 16ull << 20, 256ull << 20, 1ull << 30};
  std::vector<double> gbs, us;
  bool ok = true;
  int sms = 0;
  CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
  for (size_t nbytes : sizes) {
    uint8_t *src = nullptr, *dst = nullptr;
    CK(cudaMalloc(&src, nbytes));
    CK(cudaMalloc(&dst, nbytes));
    CK(cudaMemset(src, 0x5a, nbytes));
    CK(cudaMemset(dst, 0, nbytes));
    const size_t nvec = nbytes / 16;
    const int blocks = sms * 8, threads = 256;
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    for (int i = 0; i < 3; ++i)
      copy_kernel<<<blocks, threads>>>(reinterpret_cast<uint4*>(src), reinterpret_cast<uint4*>(dst), nvec);
    CK(cudaDeviceSynchronize());
    CK(cudaEventRecord(e0));
    for (int i = 0; i < 10; ++i)
      copy_kernel<<<blocks, threads>>>(reinterpret_cast<uint4*>(src), reinterpret_cast<uint4*>(dst), nvec);
    CK(cudaEventRecord(e1));
    CK(cudaEventSynchronize(e1));
    float ms = 0.f;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    const double sec = ms / 1e3 / 10;
    us.push_back(sec * 1e6);
    gbs.push_back(2.0 * nbytes / sec / 1e9);
    std::vector<uint8_t> head(4096), tail(4096);
    CK(cudaMemcpy(head.data(), dst, 4096, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(tail.data(), dst + nbytes - 4096, 4096, cudaMemcpyDeviceToHost));
    for (int i = 0; i < 4096; ++i) ok = ok && head[i] == 0x5a && tail[i] == 0x5a;
    CK(cudaEventDestroy(e0));
    CK(cudaEventDestroy(e1));
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
