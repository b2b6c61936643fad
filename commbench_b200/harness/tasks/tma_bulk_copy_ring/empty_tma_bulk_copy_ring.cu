// Bulk asynchronous copies global -> shared memory (the 1-D form of the tensor memory
// accelerator) through a multi-stage ring: one producer thread issues cp.async.bulk with an
// mbarrier transaction count, four consumer warps wait on the "full" barrier, read the tile and
// hand the slot back through an "empty" barrier.  Reports the aggregate load bandwidth for a
// range of grid sizes.  Prints one JSON object.
//
// No cluster multicast may be used.  Every wait must be bounded: a wait that runs out sets a bit
// in `errors`, the CTA gives copies in flight a grace period and returns.
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

constexpr uint32_t kTileBytes = 64 * 1024;
constexpr int kStages = 3;
constexpr int kConsumers = 128;
constexpr int kThreads = 32 + kConsumers;
constexpr uint32_t kPollLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbarrier_init(uint64_t* bar, uint32_t count) {
  // TODO: mbarrier.init.shared::cta.b64
}
__device__ __forceinline__ void mbarrier_arrive(uint64_t* bar) {
  // TODO: mbarrier.arrive.shared::cta.b64
}
__device__ __forceinline__ void mbarrier_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  // TODO: mbarrier.arrive.expect_tx.shared::cta.b64
}
__device__ __forceinline__ bool mbarrier_wait(uint64_t* bar, uint32_t parity) {
  // TODO: at most kPollLimit polls of mbarrier.try_wait.parity.shared::cta.b64; false when it ran out
  return false;
}
// 16-byte aligned addresses, size a multiple of 16; completion is counted on `bar` in bytes.
__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  // TODO: cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes (no multicast)
}

__host__ __device__ inline uint32_t pattern(uint64_t word) { return static_cast<uint32_t>(word * 2654435761ull + 12345u); }

__global__ void fill_kernel(uint32_t* p, size_t nwords) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nwords;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    p[i] = pattern(i);
}

// CTA b reads tiles b, b + G, b + 2G, ... (mod ntiles), `iters` of them.  Consumer c XORs word c of
// every tile; the CTA's XOR goes to out[b].
__global__ void __launch_bounds__(kThreads)
    ring_kernel(const uint8_t* __restrict__ src, uint32_t ntiles, int iters, uint32_t* out, uint32_t* errors) {
  extern __shared__ __align__(128) uint8_t tiles[];
  // TODO:
  //  * kStages "full" barriers (1 arrival + transaction bytes) and kStages "empty" barriers
  //    (kConsumers arrivals);
  //  * thread 0 is the producer: for tile i it waits for the slot to be empty (from the second lap
  //    on), arms the full barrier with kTileBytes and issues the bulk copy of tile
  //    (blockIdx.x + i * gridDim.x) % ntiles into slot i % kStages;
  //  * threads 32 .. 32 + kConsumers - 1 are consumers: wait for the slot to be full, XOR 32-bit
  //    word (threadIdx.x - 32) of the tile into a register, arrive on the empty barrier; at the
  //    end atomicXor the register into out[blockIdx.x];
  //  * a wait that runs out: bit 0 (producer) / bit 1 (consumer) of *errors, everyone leaves, about
  //    a millisecond of grace for copies in flight before returning.
}

// One tile through shared memory and back out, for a byte-exact check.
__global__ void __launch_bounds__(kThreads)
    one_tile_kernel(const uint8_t* __restrict__ src, uint8_t* dst, uint32_t* errors) {
  extern __shared__ __align__(128) uint8_t tiles[];
  // TODO: bulk-copy kTileBytes from src to shared memory, wait (bit 2 of *errors when it runs out),
  // then copy shared memory to dst with all threads.
}

int main() {
  const size_t src_bytes = 256ull << 20;
  const uint32_t ntiles = static_cast<uint32_t>(src_bytes / kTileBytes);
  const int iters = 256;
  int sms = 0;
  CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
  const size_t smem = static_cast<size_t>(kStages) * kTileBytes;
  CK(cudaFuncSetAttribute(ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  CK(cudaFuncSetAttribute(one_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kTileBytes)));
  uint8_t *src = nullptr, *one = nullptr;
  uint32_t *out = nullptr, *err = nullptr;
  CK(cudaMalloc(&src, src_bytes));
  CK(cudaMalloc(&one, kTileBytes));
  CK(cudaMalloc(&out, 4096 * sizeof(uint32_t)));
  CK(cudaMalloc(&err, sizeof(uint32_t)));
  CK(cudaMemset(err, 0, sizeof(uint32_t)));
  fill_kernel<<<sms * 4, 256>>>(reinterpret_cast<uint32_t*>(src), src_bytes / 4);
  CK(cudaDeviceSynchronize());

  bool ok = true;
  // byte-exact check of one tile (tile 5)
  one_tile_kernel<<<1, kThreads, kTileBytes>>>(src + 5ull * kTileBytes, one, err);
  CK(cudaDeviceSynchronize());
  std::vector<uint32_t> host(kTileBytes / 4);
  CK(cudaMemcpy(host.data(), one, kTileBytes, cudaMemcpyDeviceToHost));
  for (uint32_t i = 0; i < kTileBytes / 4; ++i) ok = ok && host[i] == pattern(5ull * (kTileBytes / 4) + i);

  const int grids[] = {1, 4, 16, 64, sms, 2 * sms};
  std::vector<double> gbs, us;
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  for (int g : grids) {
    ring_kernel<<<g, kThreads, smem>>>(src, ntiles, iters, out, err);  // warm-up
    CK(cudaMemset(out, 0, 4096 * sizeof(uint32_t)));
    CK(cudaEventRecord(e0));
    ring_kernel<<<g, kThreads, smem>>>(src, ntiles, iters, out, err);
    CK(cudaEventRecord(e1));
    CK(cudaEventSynchronize(e1));
    float ms = 0.f;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    us.push_back(ms * 1e3);
    gbs.push_back(static_cast<double>(g) * iters * kTileBytes / (ms / 1e3) / 1e9);
    std::vector<uint32_t> got(g);
    CK(cudaMemcpy(got.data(), out, g * sizeof(uint32_t), cudaMemcpyDeviceToHost));
    for (int b = 0; b < g; ++b) {
      uint32_t want = 0;
      for (int i = 0; i < iters; ++i) {
        const uint64_t t = (b + static_cast<uint64_t>(i) * g) % ntiles;
        for (int c = 0; c < kConsumers; ++c) want ^= pattern(t * (kTileBytes / 4) + c);
      }
      ok = ok && got[b] == want;
    }
  }
  uint32_t herr = 0;
  CK(cudaMemcpy(&herr, err, sizeof(herr), cudaMemcpyDeviceToHost));
  ok = ok && herr == 0;
  printf("{\"Correctness\": \"%s\", \"data_size_unit\": \"CTAs\", \"latency_unit\": \"us\", "
         "\"throughput_unit\": \"GB/s\", \"metrics\": [", ok ? "PASS" : "FAIL");
  for (size_t i = 0; i < gbs.size(); ++i)
    printf("%s{\"data_size\": %d, \"latency_avg\": %.2f, \"throughput_avg\": %.2f}", i ? ", " : "", grids[i], us[i],
           gbs[i]);
  printf("]}\n");
  return ok ? 0 : 1;
}
