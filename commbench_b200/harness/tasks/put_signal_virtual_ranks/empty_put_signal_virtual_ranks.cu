// One-sided transfers between pairs of ranks with a flag as the only synchronisation, in the
// two classic forms:
//   push ("put, then signal"): the producer writes its data into the consumer's buffer with
//        16-byte stores, then releases a flag; the consumer waits on the flag (acquire) and uses
//        the data;
//   pull ("signal, then get"): the producer releases a flag saying "my buffer is ready"; the
//        consumer waits on it and reads the producer's buffer itself.
// Ranks 0->1 and 2->3 are paired.  The four ranks are VIRTUAL: one cooperative launch whose
// grid is four groups of resident blocks with their own buffers; block b of the producer
// handles slice b and signals block b of the consumer, so the protocol and the memory ordering
// are those of the two-GPU kernel while nothing ever waits on another launch.
// Prints one JSON object.
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

constexpr int kWorld = 4;
constexpr int kThreads = 256;
constexpr int kMaxBlocksPerRank = 32;
constexpr uint32_t kPollLimit = 1u << 22;

struct Args {
  const uint4* src[kWorld];  // what a producer owns (only even ranks are read)
  uint4* dst[kWorld];        // where a consumer ends up with the data (only odd ranks are written)
  uint32_t* flags;           // [kWorld owner][kMaxBlocksPerRank channel]: written by the owner's partner
  uint32_t* errors;          // bit 0: a consumer's wait ran out
  size_t nvec;               // 16-byte vectors per rank
  uint32_t epoch;            // this launch signals with epoch + 1
  int pull;                  // 0: put then signal, 1: signal then get
};

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
  // TODO: st.release.sys.global.u32
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
  uint32_t v = 0;
  // TODO: ld.acquire.sys.global.u32
  return v;
}

// All threads of the block call it; true when `flag` reached `value` within kPollLimit polls of
// thread 0.
__device__ bool wait_flag(const uint32_t* flag, uint32_t value) {
  // TODO: thread 0 polls with acquire loads, the block learns the outcome through
  //       __syncthreads_and (which also orders the other threads' later reads after the acquire)
  return false;
}

// grid = kWorld * blocks_per_rank (cooperative launch: every block is resident).
__global__ void __launch_bounds__(kThreads) transfer_kernel(Args a, int blocks_per_rank) {
  const int rank = blockIdx.x / blocks_per_rank, ch = blockIdx.x % blocks_per_rank;
  const bool producer = (rank % 2) == 0;
  const int partner = producer ? rank + 1 : rank - 1;
  const size_t per = (a.nvec + blocks_per_rank - 1) / blocks_per_rank;
  const size_t lo = per * ch < a.nvec ? per * ch : a.nvec, hi = lo + per < a.nvec ? lo + per : a.nvec;
  uint32_t* consumer_flag = a.flags + (producer ? partner : rank) * kMaxBlocksPerRank + ch;
  // TODO: producer, push: copy slice [lo, hi) of src[rank] into dst[partner], __syncthreads(),
  //       thread 0 releases consumer_flag = epoch + 1.  producer, pull: thread 0 releases the flag
  //       at once (the source was written before the launch).  consumer: wait_flag (bit 0 of
  //       *a.errors and return when it runs out); pull only: copy the slice of src[partner] into
  //       dst[rank] itself.
}

__global__ void fill_kernel(uint32_t* p, size_t nwords, uint32_t seed) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nwords;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    p[i] = static_cast<uint32_t>(i) * 2654435761u + seed;
}

int main() {
  int coop = 0, sms = 0, per_sm = 0;
  CK(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, 0));
  CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
  CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, transfer_kernel, kThreads, 0));
  if (!coop || per_sm < 1) {
    printf("{\"Correctness\": \"SKIP\", \"reason\": \"no cooperative launch\"}\n");
    return 0;
  }
  int blocks_per_rank = sms * per_sm / kWorld;
  if (blocks_per_rank > kMaxBlocksPerRank) blocks_per_rank = kMaxBlocksPerRank;
  const size_t sizes[] = {4096, 1u << 20, 64u << 20};  // bytes per rank
  const size_t max_bytes = sizes[2];
  Args a{};
  uint4* src[kWorld];
  uint4* dst[kWorld];
  for (int r = 0; r < kWorld; ++r) {
    CK(cudaMalloc(&src[r], max_bytes));
    CK(cudaMalloc(&dst[r], max_bytes));
    a.src[r] = src[r];
    a.dst[r] = dst[r];
  }
  CK(cudaMalloc(&a.flags, sizeof(uint32_t) * kWorld * kMaxBlocksPerRank));
  CK(cudaMemset(a.flags, 0, sizeof(uint32_t) * kWorld * kMaxBlocksPerRank));
  CK(cudaMalloc(&a.errors, sizeof(uint32_t)));
  CK(cudaMemset(a.errors, 0, sizeof(uint32_t)));
  bool ok = true;
  uint32_t epoch = 0;
  std::vector<double> us_push, us_pull;
  std::vector<uint32_t> host(max_bytes / 4);
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  for (size_t bytes : sizes) {
    a.nvec = bytes / 16;
    for (int pull = 0; pull < 2; ++pull) {
      a.pull = pull;
      for (int round = 0; round < 2; ++round) {  // repeated calls exercise the epochs
        const uint32_t seed = 1000u * pull + 10u * round + 1u;
        for (int r = 0; r < kWorld; r += 2) fill_kernel<<<sms, 256>>>(reinterpret_cast<uint32_t*>(src[r]), bytes / 4, seed + r);
        for (int r = 1; r < kWorld; r += 2) CK(cudaMemsetAsync(dst[r], 0, bytes));
        a.epoch = epoch++;
        void* params[] = {&a, &blocks_per_rank};
        CK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(transfer_kernel), dim3(kWorld * blocks_per_rank),
                                       dim3(kThreads), params, 0, nullptr));
        CK(cudaDeviceSynchronize());
        for (int r = 1; r < kWorld; r += 2) {
          CK(cudaMemcpy(host.data(), dst[r], bytes, cudaMemcpyDeviceToHost));
          for (size_t i = 0; i < bytes / 4; ++i)
            ok = ok && host[i] == static_cast<uint32_t>(i) * 2654435761u + seed + (r - 1);
        }
      }
      const int iters = 20;
      CK(cudaEventRecord(e0));
      for (int it = 0; it < iters; ++it) {
        a.epoch = epoch++;
        void* params[] = {&a, &blocks_per_rank};
        CK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(transfer_kernel), dim3(kWorld * blocks_per_rank),
                                       dim3(kThreads), params, 0, nullptr));
      }
      CK(cudaEventRecord(e1));
      CK(cudaEventSynchronize(e1));
      float ms = 0.f;
      CK(cudaEventElapsedTime(&ms, e0, e1));
      (pull ? us_pull : us_push).push_back(ms * 1e3 / iters);
    }
  }
  uint32_t herr = 0;
  CK(cudaMemcpy(&herr, a.errors, sizeof(herr), cudaMemcpyDeviceToHost));
  ok = ok && herr == 0;
  printf("{\"Correctness\": \"%s\", \"virtual_ranks\": %d, \"blocks_per_rank\": %d, \"data_size_unit\": \"KB\", "
         "\"latency_unit\": \"us\", \"throughput_unit\": \"GB/s\", \"metrics\": [",
         ok ? "PASS" : "FAIL", kWorld, blocks_per_rank);
  for (size_t i = 0; i < us_push.size(); ++i) {
    const double bytes = static_cast<double>(sizes[i]);
    printf("%s{\"data_size\": %.1f, \"latency_avg\": %.3f, \"pull_latency_avg\": %.3f, \"throughput_avg\": %.3f}",
           i ? ", " : "", bytes / 1024.0, us_push[i], us_pull[i], 2.0 * bytes / (us_push[i] * 1e-6) / 1e9);
  }
  printf("]}\n");
  return ok ? 0 : 1;
}
