// Expert-parallel dispatch layout: from the router's top-k expert ids per token compute how many
// tokens each expert receives, which ranks each token must be sent to (a token goes to a rank
// once, however many of its experts live there) and how many tokens each rank receives.
// Prints one JSON object.
//
// Same exercise as the reference's datasets/example042_deepep_dispatch_layout (kernel :48-86,
// CPU reference :208-234, correctness grid T x K x R with three routing patterns :401-410, timing
// T = 1k..64k :419-424).
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

constexpr int kMaxExperts = 1024;
constexpr int kMaxRanks = 8;
constexpr int kThreads = 256;

// topk_idx [T, K] int64, -1 = slot unused.  Experts are split evenly over ranks in order.
// Outputs must be zeroed by the caller.
__global__ void __launch_bounds__(kThreads)
    dispatch_layout_kernel(const int64_t* __restrict__ topk_idx, int T, int K, int E, int R,
                           int* __restrict__ tokens_per_expert, int* __restrict__ tokens_per_rank,
                           uint8_t* __restrict__ is_token_in_rank) {
  __shared__ int s_expert[kMaxExperts];
  __shared__ int s_rank[kMaxRanks];
  for (int i = threadIdx.x; i < E; i += blockDim.x) s_expert[i] = 0;
  if (threadIdx.x < kMaxRanks) s_rank[threadIdx.x] = 0;
  __syncthreads();
  const int per_rank = E / R;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x) {
    uint32_t ranks = 0;
    for (int k = 0; k < K; ++k) {
      const int64_t e = topk_idx[static_cast<size_t>(t) * K + k];
      if (e < 0 || e >= E) continue;
      atomicAdd(&s_expert[e], 1);
      ranks |= 1u << (static_cast<int>(e) / per_rank);
    }
    for (int r = 0; r < R; ++r) {
      const bool in = (ranks >> r) & 1u;
      is_token_in_rank[static_cast<size_t>(t) * R + r] = in ? 1 : 0;
      if (in) atomicAdd(&s_rank[r], 1);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x)
    if (s_expert[i] != 0) atomicAdd(&tokens_per_expert[i], s_expert[i]);
  if (threadIdx.x < R && s_rank[threadIdx.x] != 0) atomicAdd(&tokens_per_rank[threadIdx.x], s_rank[threadIdx.x]);
}

// pattern 0: pseudo-random distinct experts; 1: everything on the first rank's experts (dedup case);
// 2: round-robin with some slots unused (-1).
static void make_routing(std::vector<int64_t>& idx, int T, int K, int E, int R, int pattern) {
  idx.assign(static_cast<size_t>(T) * K, -1);
  uint64_t s = 0x9e3779b97f4a7c15ull ^ (static_cast<uint64_t>(T) * 131 + K * 17 + R);
  for (int t = 0; t < T; ++t)
    for (int k = 0; k < K; ++k) {
      s = s * 6364136223846793005ull + 1442695040888963407ull;
      int64_t e;
      if (pattern == 0) e = static_cast<int64_t>(((s >> 33) % (E / K)) * K + k);        // distinct per slot
      else if (pattern == 1) e = k % (E / R);
      else e = ((t + k) % 3 == 0) ? -1 : static_cast<int64_t>((static_cast<int64_t>(t) * K + k) % E);
      idx[static_cast<size_t>(t) * K + k] = e;
    }
}

static void cpu_layout(const std::vector<int64_t>& idx, int T, int K, int E, int R, std::vector<int>& pe,
                       std::vector<int>& pr, std::vector<uint8_t>& in) {
  pe.assign(E, 0);
  pr.assign(R, 0);
  in.assign(static_cast<size_t>(T) * R, 0);
  for (int t = 0; t < T; ++t) {
    for (int k = 0; k < K; ++k) {
      const int64_t e = idx[static_cast<size_t>(t) * K + k];
      if (e < 0) continue;
      pe[e]++;
      in[static_cast<size_t>(t) * R + e / (E / R)] = 1;
    }
    for (int r = 0; r < R; ++r) pr[r] += in[static_cast<size_t>(t) * R + r];
  }
}

struct Buffers {
  int64_t* idx = nullptr;
  int *pe = nullptr, *pr = nullptr;
  uint8_t* in = nullptr;
};

static cudaError_t launch(const Buffers& b, int T, int K, int E, int R, int sms) {
  cudaError_t e = cudaMemsetAsync(b.pe, 0, E * sizeof(int));
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(b.pr, 0, kMaxRanks * sizeof(int));
  if (e != cudaSuccess) return e;
  int blocks = (T + kThreads - 1) / kThreads;
  if (blocks > sms * 2) blocks = sms * 2;
  dispatch_layout_kernel<<<blocks, kThreads>>>(b.idx, T, K, E, R, b.pe, b.pr, b.in);
  return cudaGetLastError();
}

int main() {
  int sms = 0;
  CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
  const int maxT = 65536, maxK = 8;
  Buffers b;
  CK(cudaMalloc(&b.idx, static_cast<size_t>(maxT) * maxK * sizeof(int64_t)));
  CK(cudaMalloc(&b.pe, kMaxExperts * sizeof(int)));
  CK(cudaMalloc(&b.pr, kMaxRanks * sizeof(int)));
  CK(cudaMalloc(&b.in, static_cast<size_t>(maxT) * kMaxRanks));
  bool ok = true;
  std::vector<int64_t> idx;
  std::vector<int> pe, pr, gpe, gpr;
  std::vector<uint8_t> in, gin;
  const int E = 64;
  for (int T : {257, 1024, 4096})
    for (int K : {1, 2, 4, 8})
      for (int R : {1, 2, 4, 8})
        for (int pattern = 0; pattern < 3; ++pattern) {
          make_routing(idx, T, K, E, R, pattern);
          cpu_layout(idx, T, K, E, R, pe, pr, in);
          CK(cudaMemcpy(b.idx, idx.data(), idx.size() * sizeof(int64_t), cudaMemcpyHostToDevice));
          CK(launch(b, T, K, E, R, sms));
          CK(cudaDeviceSynchronize());
          gpe.resize(E);
          gpr.resize(R);
          gin.resize(static_cast<size_t>(T) * R);
          CK(cudaMemcpy(gpe.data(), b.pe, E * sizeof(int), cudaMemcpyDeviceToHost));
          CK(cudaMemcpy(gpr.data(), b.pr, R * sizeof(int), cudaMemcpyDeviceToHost));
          CK(cudaMemcpy(gin.data(), b.in, gin.size(), cudaMemcpyDeviceToHost));
          ok = ok && gpe == pe && gpr == pr && gin == in;
        }
  // timing: 32 experts, top-8, 8 ranks
  std::vector<double> us;
  const int sizes[] = {1024, 4096, 16384, 65536};
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  for (int T : sizes) {
    make_routing(idx, T, 8, 32, 8, 0);
    CK(cudaMemcpy(b.idx, idx.data(), idx.size() * sizeof(int64_t), cudaMemcpyHostToDevice));
    for (int i = 0; i < 20; ++i) CK(launch(b, T, 8, 32, 8, sms));
    CK(cudaEventRecord(e0));
    for (int i = 0; i < 100; ++i) CK(launch(b, T, 8, 32, 8, sms));
    CK(cudaEventRecord(e1));
    CK(cudaEventSynchronize(e1));
    float ms = 0.f;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    us.push_back(ms * 1e3 / 100);
  }
  printf("{\"Correctness\": \"%s\", \"data_size_unit\": \"tokens\", \"latency_unit\": \"us\", "
         "\"throughput_unit\": \"Mtokens/s\", \"metrics\": [", ok ? "PASS" : "FAIL");
  for (size_t i = 0; i < us.size(); ++i)
    printf("%s{\"data_size\": %d, \"latency_avg\": %.3f, \"throughput_avg\": %.3f}", i ? ", " : "", sizes[i], us[i],
           sizes[i] / us[i]);
  printf("]}\n");
  return ok ? 0 : 1;
}
