// Stable sort of MoE selections by expert (see expert_sort.h).  Three small kernels:
// per-expert scan (slot of every selection inside its expert + counts), exclusive prefix
// over the counts, scatter.  The deterministic slot scan is the idea of the reference's
// deterministic dispatch prologue (datasets/example078_deepep_jit_dispatch_deterministic_prologue/
// nv/empty_deepep_jit_dispatch_deterministic_prologue.cu:12-55).
#include "expert_sort.h"

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>

namespace cb {
void set_last_error(const std::string& s);

// One warp per expert walks all selections in order.
__global__ void esort_slot_kernel(const int* __restrict__ topk_idx, int n_pairs, int E,
                                  int* __restrict__ slot, int* __restrict__ counts) {
  const int e = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (e >= E) return;
  int running = 0;
  for (int base = 0; base < n_pairs; base += 32) {
    const int i = base + lane;
    const bool hit = i < n_pairs && topk_idx[i] == e;
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (hit) slot[i] = running + __popc(m & ((1u << lane) - 1u));
    running += __popc(m);
  }
  if (lane == 0) counts[e] = running;
}

// Exclusive prefix sum of counts[E] (E <= 1024), one CTA of 1024 threads.
__global__ void esort_prefix_kernel(const int* __restrict__ counts, int E, int* __restrict__ base) {
  __shared__ int sh[1024];
  const int t = threadIdx.x;
  sh[t] = t < E ? counts[t] : 0;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const int v = t >= o ? sh[t - o] : 0;
    __syncthreads();
    sh[t] += v;
    __syncthreads();
  }
  if (t < E) base[t] = sh[t] - counts[t];
}

__global__ void esort_scatter_kernel(const int* __restrict__ topk_idx, const int* __restrict__ slot,
                                     const int* __restrict__ base, int n_pairs, int E,
                                     int* __restrict__ sorted_pair) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  const int e = topk_idx[i];
  if (e < 0 || e >= E) return;
  sorted_pair[base[e] + slot[i]] = i;
}

static int run_expert_sort(const int* topk_idx, int n_pairs, int E, int* scratch, int* sorted_pair,
                           int* counts, cudaStream_t st) {
  int* slot = scratch;            // [n_pairs]
  int* base = scratch + n_pairs;  // [E]
  esort_slot_kernel<<<(E * 32 + 255) / 256, 256, 0, st>>>(topk_idx, n_pairs, E, slot, counts);
  esort_prefix_kernel<<<1, 1024, 0, st>>>(counts, E, base);
  esort_scatter_kernel<<<(n_pairs + 255) / 256, 256, 0, st>>>(topk_idx, slot, base, n_pairs, E,
                                                              sorted_pair);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(std::string("expert sort launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

// Scratch of the allocation-free entry point.  In host code this name is only a handle for
// cudaGetSymbolAddress: it is NOT a device address and must never be passed to a kernel.
static __device__ __align__(256) int
    g_esort_static_scratch[CB_EXPERT_SORT_STATIC_MAX_PAIRS + CB_EXPERT_SORT_STATIC_MAX_EXPERTS];

static constexpr int kMaxDevices = 64;
static int* g_esort_scratch_addr[kMaxDevices] = {};  // device address of the array, per device
static std::mutex g_esort_mutex;

// Device address of the static scratch on the CURRENT device (looked up once per device).
static int* esort_static_scratch() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_last_error("expert sort (no-alloc): cannot identify the current device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_esort_mutex);
  if (g_esort_scratch_addr[dev] == nullptr) {
    int* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_esort_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_last_error(std::string("expert sort (no-alloc): cudaGetSymbolAddress: ") +
                     cudaGetErrorString(e));
      return nullptr;
    }
    g_esort_scratch_addr[dev] = p;
  }
  return g_esort_scratch_addr[dev];
}

}  // namespace cb

using namespace cb;

extern "C" {

int cb_moe_expert_sort_noalloc(const void* topk_idx, int n_pairs, int E, void* sorted_pair,
                               void* counts, void* stream) {
  if (n_pairs < 1 || E < 1) {
    set_last_error("expert sort (no-alloc): need n_pairs >= 1 and E >= 1");
    return -1;
  }
  if (n_pairs > CB_EXPERT_SORT_STATIC_MAX_PAIRS || E > CB_EXPERT_SORT_STATIC_MAX_EXPERTS) {
    set_last_error("expert sort (no-alloc): problem exceeds the built-in scratch (" +
                   std::to_string(CB_EXPERT_SORT_STATIC_MAX_PAIRS) + " selections, " +
                   std::to_string(CB_EXPERT_SORT_STATIC_MAX_EXPERTS) +
                   " experts); use cb_moe_expert_sort with your own scratch");
    return -1;
  }
  int* scratch = esort_static_scratch();
  if (scratch == nullptr) return -1;
  return run_expert_sort(static_cast<const int*>(topk_idx), n_pairs, E, scratch,
                         static_cast<int*>(sorted_pair), static_cast<int*>(counts),
                         static_cast<cudaStream_t>(stream));
}

int cb_moe_expert_sort(const void* topk_idx, int n_pairs, int E, void* scratch, void* sorted_pair,
                       void* counts, void* stream) {
  if (n_pairs < 1 || E < 1 || E > 1024) {
    set_last_error("expert sort: need n_pairs >= 1 and 1 <= E <= 1024");
    return -1;
  }
  if (scratch == nullptr) {
    set_last_error("expert sort: scratch of (n_pairs + E) ints required");
    return -1;
  }
  return run_expert_sort(static_cast<const int*>(topk_idx), n_pairs, E, static_cast<int*>(scratch),
                         static_cast<int*>(sorted_pair), static_cast<int*>(counts),
                         static_cast<cudaStream_t>(stream));
}

}  // extern "C"
