// One-shot "pull" all-reduce among W ranks with the rank barrier folded into the kernel:
// every rank signals "my input is ready" into a flag matrix with a release store, waits with
// acquire loads until every peer has signalled, then reads all W inputs, adds them in rank
// order and writes its own output; a second barrier keeps any rank from leaving (and its input
// from being reused) while a peer still reads.  Here the W ranks are VIRTUAL: one cooperative
// launch whose grid is W groups of blocks, all resident at once, each group working on its own
// buffers - the protocol, the flags and the memory ordering are those of the multi-GPU kernel,
// but nothing ever waits on a different launch.  Prints one JSON object.
//
// Reference counterpart: datasets/example105_sglang_custom_allreduce_easy (one-shot pull kernel
// with signal/wait semaphores :49-111) and datasets/example017_intranode_gpu_barrier (flag-matrix
// barrier :38-53), with system-scope acquire/release as in
// datasets/example073_GPU_p2p_pingpong_latency (:30-43).  Every wait is bounded.
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
  const float* in[kWorld];   // input of every virtual rank
  float* out[kWorld];        // output of every virtual rank
  uint32_t* flags;           // [kWorld dst][kMaxBlocksPerRank channel][kWorld src]
  uint32_t* errors;          // bit 0: a start-barrier wait ran out, bit 1: an end-barrier wait
  size_t n;                  // elements per rank
  uint32_t epoch;            // the two barriers of this launch use epoch + 1 and epoch + 2
};

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
  // --- solution: st.release.sys.global.u32
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
  // --- end solution
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
  uint32_t v = 0;
  // --- solution: ld.acquire.sys.global.u32
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  // --- end solution
  return v;
}

// Barrier among block `ch` of every virtual rank.  Returns false when a peer did not show up
// within kPollLimit polls.  All threads of the block call it.
__device__ bool rank_barrier(uint32_t* flags, int rank, int ch, uint32_t value) {
  // --- solution else: return false;: __syncthreads(); thread t < kWorld stores `value` (release) into word
  //     [dst = t][ch][src = rank] and then polls word [dst = rank][ch][src = t] (acquire) until it
  //     is >= value, at most kPollLimit times; the block agrees on the outcome with
  //     __syncthreads_and
  __syncthreads();
  bool ok = true;
  if (threadIdx.x < kWorld) {
    const int t = threadIdx.x;
    store_release_sys(flags + (static_cast<size_t>(t) * kMaxBlocksPerRank + ch) * kWorld + rank, value);
    const uint32_t* mine = flags + (static_cast<size_t>(rank) * kMaxBlocksPerRank + ch) * kWorld + t;
    ok = false;
    for (uint32_t i = 0; i < kPollLimit; ++i) {
      if (load_acquire_sys(mine) >= value) {
        ok = true;
        break;
      }
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
  // --- end solution
}

// grid = kWorld * blocks_per_rank (cooperative launch: every block is resident).
__global__ void __launch_bounds__(kThreads) allreduce_kernel(Args a, int blocks_per_rank) {
  const int rank = blockIdx.x / blocks_per_rank, ch = blockIdx.x % blocks_per_rank;
  // --- solution: start barrier (epoch + 1; on failure set bit 0 of *a.errors and return); then
  //     this block's slice of the elements: out[rank][i] = in[0][i] + in[1][i] + ... in rank
  //     order (every rank then holds the same bits); end barrier (epoch + 2; bit 1 on failure)
  if (!rank_barrier(a.flags, rank, ch, a.epoch + 1)) {
    if (threadIdx.x == 0) atomicOr(a.errors, 1u);
    return;
  }
  const size_t per = (a.n + blocks_per_rank - 1) / blocks_per_rank;
  const size_t lo = per * ch, hi = lo + per < a.n ? lo + per : a.n;
  for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    float acc = a.in[0][i];
#pragma unroll
    for (int r = 1; r < kWorld; ++r) acc += a.in[r][i];
    a.out[rank][i] = acc;
  }
  if (!rank_barrier(a.flags, rank, ch, a.epoch + 2)) {
    if (threadIdx.x == 0) atomicOr(a.errors, 2u);
  }
  // --- end solution
}

__global__ void fill_kernel(float* p, size_t n, int rank, int round) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    p[i] = static_cast<float>(static_cast<int>((i * 7 + rank * 13 + round * 5) % 31) - 15);
}

static float expected(size_t i, int round) {
  float s = 0.f;
  for (int r = 0; r < kWorld; ++r) s += static_cast<float>(static_cast<int>((i * 7 + r * 13 + round * 5) % 31) - 15);
  return s;
}

int main() {
  int coop = 0, sms = 0, per_sm = 0;
  CK(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, 0));
  CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
  CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_kernel, kThreads, 0));
  if (!coop || per_sm < 1) {
    printf("{\"Correctness\": \"SKIP\", \"reason\": \"no cooperative launch\"}\n");
    return 0;
  }
  int blocks_per_rank = sms * per_sm / kWorld;
  if (blocks_per_rank > kMaxBlocksPerRank) blocks_per_rank = kMaxBlocksPerRank;
  const size_t sizes[] = {1000, 1u << 16, 1u << 22};
  const size_t max_n = sizes[2];
  Args a{};
  float* in[kWorld];
  float* out[kWorld];
  for (int r = 0; r < kWorld; ++r) {
    CK(cudaMalloc(&in[r], max_n * sizeof(float)));
    CK(cudaMalloc(&out[r], max_n * sizeof(float)));
    a.in[r] = in[r];
    a.out[r] = out[r];
  }
  CK(cudaMalloc(&a.flags, sizeof(uint32_t) * kWorld * kMaxBlocksPerRank * kWorld));
  CK(cudaMemset(a.flags, 0, sizeof(uint32_t) * kWorld * kMaxBlocksPerRank * kWorld));
  CK(cudaMalloc(&a.errors, sizeof(uint32_t)));
  CK(cudaMemset(a.errors, 0, sizeof(uint32_t)));
  bool ok = true;
  uint32_t epoch = 0;
  std::vector<double> us;
  std::vector<float> host(max_n);
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  for (size_t n : sizes) {
    a.n = n;
    for (int round = 0; round < 3; ++round) {  // repeated calls exercise the epoch counters
      for (int r = 0; r < kWorld; ++r) fill_kernel<<<sms, 256>>>(in[r], n, r, round);
      a.epoch = epoch;
      epoch += 2;
      void* params[] = {&a, &blocks_per_rank};
      CK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(allreduce_kernel), dim3(kWorld * blocks_per_rank),
                                     dim3(kThreads), params, 0, nullptr));
      CK(cudaDeviceSynchronize());
      for (int r = 0; r < kWorld; ++r) {
        CK(cudaMemcpy(host.data(), out[r], n * sizeof(float), cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < n; ++i) ok = ok && host[i] == expected(i, round);
      }
    }
    const int iters = 20;
    CK(cudaEventRecord(e0));
    for (int it = 0; it < iters; ++it) {
      a.epoch = epoch;
      epoch += 2;
      void* params[] = {&a, &blocks_per_rank};
      CK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(allreduce_kernel), dim3(kWorld * blocks_per_rank),
                                     dim3(kThreads), params, 0, nullptr));
    }
    CK(cudaEventRecord(e1));
    CK(cudaEventSynchronize(e1));
    float ms = 0.f;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    us.push_back(ms * 1e3 / iters);
  }
  uint32_t herr = 0;
  CK(cudaMemcpy(&herr, a.errors, sizeof(herr), cudaMemcpyDeviceToHost));
  ok = ok && herr == 0;
  printf("{\"Correctness\": \"%s\", \"virtual_ranks\": %d, \"blocks_per_rank\": %d, \"data_size_unit\": \"KB\", "
         "\"latency_unit\": \"us\", \"throughput_unit\": \"GB/s\", \"metrics\": [",
         ok ? "PASS" : "FAIL", kWorld, blocks_per_rank);
  for (size_t i = 0; i < us.size(); ++i) {
    const double bytes = static_cast<double>(sizes[i]) * sizeof(float);
    printf("%s{\"data_size\": %.1f, \"latency_avg\": %.3f, \"throughput_avg\": %.3f}", i ? ", " : "", bytes / 1024.0,
           us[i], bytes * kWorld * (kWorld + 1) / (us[i] * 1e-6) / 1e9);
  }
  printf("]}\n");
  return ok ? 0 : 1;
}
