// Expert-parallel MoE kernels (everything except the grouped GEMMs):
//   router (softmax top-k, renormalised), dispatch layout, deterministic slot
//   assignment, the global row plan, the fp8-quantising dispatch push with
//   per-expert arrival counters, the dequantising receive, SwiGLU, and the
//   weighted combine reduction.
//
// Where the reference has the same capability:
//   layout        datasets/example042_deepep_dispatch_layout/nv/empty_deepep_dispatch_layout.cu:48-86
//   notify/prefix datasets/example047_deepep_intranode_notify_dispatch/nv/
//                 empty_deepep_intranode_notify_dispatch.cu:81-159 (count exchange + prefix matrices)
//   deterministic datasets/example078_deepep_jit_dispatch_deterministic_prologue/nv/
//   slots         empty_deepep_jit_dispatch_deterministic_prologue.cu:12-55
//   payload       datasets/example080_deepep_jit_dispatch_payload/nv/empty_deepep_jit_dispatch_payload.cu:241-256,
//                 datasets/example056_thunderkitten_moe_dispatch_gemm_easy/nv/
//                 empty_thunderkitten_moe_dispatch_gemm.cu:164-202 (per-row-block arrival counters)
//   combine       datasets/example082_deepep_jit_combine/nv/empty_deepep_jit_combine.cu:15-67,
//                 datasets/example083_deepep_jit_combine_reduce_epilogue/nv/
//                 empty_deepep_jit_combine_reduce_epilogue.cu:12-53
//
// Design differences: the destination layout is expert-major with every expert's
// rows padded to a multiple of 128 so the grouped tcgen05 GEMM can tile it
// directly; row positions come from an all-gathered count matrix, so no CPU
// synchronisation sits on the path; arrival is tracked per expert, which lets
// the receiver start on an expert as soon as its rows are in.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../prim/barrier.cuh"
#include "../prim/pdl.cuh"

namespace cb {
void set_last_error(const std::string& s);

enum : uint32_t { PH_MOE_ARRIVE = 48, PH_MOE_COMBINE = 49 };

// ------------------------------------------------------------------- router
// One warp per token: softmax over E logits, top-K by repeated arg-max,
// weights renormalised to sum to 1.  E <= 1024.
__global__ void router_topk_kernel(const float* __restrict__ logits, int T, int E, int K,
                                   int* __restrict__ topk_idx, float* __restrict__ topk_w) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* row = logits + static_cast<size_t>(warp) * E;
  float v[32];
  const int per = (E + 31) / 32;
  float mx = -INFINITY;
  for (int i = 0; i < per; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int i = 0; i < per; ++i) {
    v[i] = (i * 32 + lane) < E ? __expf(v[i] - mx) : -1.f;
    if (v[i] > 0.f) sum += v[i];
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  float picked_sum = 0.f;
  float my_w = 0.f;
  int my_e = -1;
  for (int k = 0; k < K; ++k) {
    float best = -1.f;
    int best_e = 0x7fffffff;
    for (int i = 0; i < per; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > best) {
        best = v[i];
        best_e = e;
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {  // ties go to the lower expert id
        best = ob;
        best_e = oe;
      }
    }
    if ((best_e & 31) == lane) v[best_e >> 5] = -1.f;  // remove the winner
    picked_sum += best;
    if (lane == k) {
      my_w = best;
      my_e = best_e;
    }
  }
  if (lane < K) {
    topk_idx[static_cast<size_t>(warp) * K + lane] = my_e;
    topk_w[static_cast<size_t>(warp) * K + lane] = my_w / picked_sum;
  }
  (void)sum;  // softmax denominator cancels in the renormalisation
}

// ------------------------------------------------------------ dispatch layout
// num_tokens_per_expert[E], num_tokens_per_rank[R] (a token counts once per rank),
// is_token_in_rank[T,R].  One thread per token; counters by atomics (the result is
// order-independent).  Negative expert ids are skipped.
__global__ void dispatch_layout_kernel(const int* __restrict__ topk_idx, int T, int K, int R, int E,
                                       int* num_tokens_per_expert, int* num_tokens_per_rank,
                                       unsigned char* is_token_in_rank) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const int epr = E / R;
  unsigned seen = 0;
  for (int k = 0; k < K; ++k) {
    const int e = topk_idx[static_cast<size_t>(t) * K + k];
    if (e < 0 || e >= E) continue;
    atomicAdd(num_tokens_per_expert + e, 1);
    seen |= 1u << (e / epr);
  }
  for (int r = 0; r < R; ++r) {
    const bool in = (seen >> r) & 1u;
    if (is_token_in_rank != nullptr) is_token_in_rank[static_cast<size_t>(t) * R + r] = in;
    if (in) atomicAdd(num_tokens_per_rank + r, 1);
  }
}

// -------------------------------------------------- deterministic slot assignment
// One CTA per expert: slot[i] = number of earlier selections of the same expert; also yields
// counts[e].  The T*K selections are cut into one contiguous chunk per warp; a first pass
// counts each chunk's hits, a prefix over the warps gives every chunk its starting slot, a
// second pass (the list is cache resident) writes the slots.  The order is a pure function of
// topk_idx, so repeated runs place every row identically.
constexpr int kSlotWarps = 16;
__global__ void __launch_bounds__(kSlotWarps * 32)
    moe_slot_kernel(const int* __restrict__ topk_idx, int n_pairs, int E, int* __restrict__ slot,
                    int* __restrict__ counts) {
  pdl_wait();                // chained with programmatic dependent launch: see prim/pdl.cuh
  pdl_launch_dependents();
  __shared__ int chunk_hits[kSlotWarps];
  const int e = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_warp = ((n_pairs + kSlotWarps - 1) / kSlotWarps + 31) / 32 * 32;
  const int begin = min(warp * per_warp, n_pairs), end = min(begin + per_warp, n_pairs);
  int hits = 0;
#pragma unroll 4
  for (int base = begin; base < end; base += 32) {
    const int i = base + lane;
    hits += (i < end && topk_idx[i] == e) ? 1 : 0;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) hits += __shfl_xor_sync(0xffffffffu, hits, o);
  if (lane == 0) chunk_hits[warp] = hits;
  __syncthreads();
  int running = 0;
  for (int w = 0; w < warp; ++w) running += chunk_hits[w];
  if (threadIdx.x == 0) {
    int total = 0;
    for (int w = 0; w < kSlotWarps; ++w) total += chunk_hits[w];
    counts[e] = total;
  }
  for (int base = begin; base < end; base += 32) {
    const int i = base + lane;
    const bool hit = i < end && topk_idx[i] == e;
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (hit) slot[i] = running + __popc(m & ((1u << lane) - 1u));
    running += __popc(m);
  }
}

// ---------------------------------------------------------------------- plan
// From the all-gathered count matrix counts_all[W][E] every rank derives the same
// global placement.  For destination rank d and its local expert j (global e = d*El+j):
//   rows(d,j)       = sum_s counts_all[s][e]
//   base(d,j)       = sum_{j'<j} round_up(rows(d,j'), 128)
//   row of source s = base(d,j) + sum_{s'<s} counts_all[s'][e]
// Outputs for THIS rank:
//   send_row_base[E]    first destination row of my selections of expert e (at rank e/El)
//   src_pair_base[E]    first position of expert e in my expert-sorted pair list
//   recv_expected[El]   rows that will arrive for my local expert j
//   recv_base[El+1]     padded first row of my local expert j (last = total padded rows)
//   mblk_expert[...]    local expert of each 128-row block of my receive buffer
//   n_mblocks[1]
// One CTA; E <= 1024.
// The plan itself, run by one whole CTA; rows_sh / base_sh: 1024 ints of shared memory each.
__device__ __forceinline__ void moe_plan_body(const int* __restrict__ counts_all, int W, int E,
                                              int rank, int* send_row_base, int* src_pair_base,
                                              int* recv_expected, int* recv_base,
                                              int* mblk_expert, int* n_mblocks, int max_recv_rows,
                                              uint32_t* status, int* rows_sh, int* base_sh) {
  const int El = E / W;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int r = 0;
    for (int s = 0; s < W; ++s) r += counts_all[s * E + e];
    rows_sh[e] = r;
  }
  __syncthreads();
  if (threadIdx.x < W) {
    const int d = threadIdx.x;
    int acc = 0;
    for (int j = 0; j < El; ++j) {
      base_sh[d * El + j] = acc;
      acc += (rows_sh[d * El + j] + 127) / 128 * 128;
    }
    if (d == rank) {
      recv_base[El] = acc;
      n_mblocks[0] = acc / 128;
      if (acc > max_recv_rows) report_status(status, CB_BAD_ARGUMENT, PH_MOE_ARRIVE, 0xffff);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int before = 0;
    for (int s = 0; s < rank; ++s) before += counts_all[s * E + e];
    send_row_base[e] = base_sh[e] + before;
  }
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      src_pair_base[e] = acc;
      acc += counts_all[rank * E + e];
    }
  }
  for (int j = threadIdx.x; j < El; j += blockDim.x) {
    recv_expected[j] = rows_sh[rank * El + j];
    recv_base[j] = base_sh[rank * El + j];
  }
  __syncthreads();
  for (int j = threadIdx.x; j < El; j += blockDim.x) {
    const int b0 = base_sh[rank * El + j] / 128;
    const int nb = (rows_sh[rank * El + j] + 127) / 128;
    for (int b = 0; b < nb; ++b)
      if ((b0 + b) * 128 < max_recv_rows) mblk_expert[b0 + b] = j;
  }
}

__global__ void moe_plan_kernel(const int* __restrict__ counts_all, int W, int E, int rank,
                                int* send_row_base, int* src_pair_base, int* recv_expected,
                                int* recv_base, int* mblk_expert, int* n_mblocks,
                                int max_recv_rows, uint32_t* status) {
  pdl_wait();                // chained with programmatic dependent launch: see prim/pdl.cuh
  pdl_launch_dependents();
  __shared__ int rows_sh[1024];   // rows(d,j) for every global expert
  __shared__ int base_sh[1024];   // base(d,j)
  moe_plan_body(counts_all, W, E, rank, send_row_base, src_pair_base, recv_expected, recv_base,
                mblk_expert, n_mblocks, max_recv_rows, status, rows_sh, base_sh);
}

// Plan and pair sort in one launch.  The sort needs only this rank's own row of the count
// matrix (src_pair_base = exclusive prefix of it), so every CTA rebuilds that prefix in shared
// memory - E <= 1024 words - and places its 256 pairs; CTA 0 also runs the plan.
__global__ void __launch_bounds__(256)
    moe_plan_sort_kernel(const int* __restrict__ counts_all, int W, int E, int rank,
                         const int* __restrict__ topk_idx, const int* __restrict__ slot,
                         int n_pairs, int* __restrict__ sorted_pair, int* send_row_base,
                         int* src_pair_base, int* recv_expected, int* recv_base,
                         int* mblk_expert, int* n_mblocks, int max_recv_rows, uint32_t* status) {
  pdl_wait();                // chained with programmatic dependent launch: see prim/pdl.cuh
  pdl_launch_dependents();
  __shared__ int pre_sh[1024];    // exclusive prefix of my counts
  __shared__ int rows_sh[1024];
  __shared__ int base_sh[1024];
  const int* __restrict__ mine = counts_all + static_cast<size_t>(rank) * E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) pre_sh[e] = mine[e];
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    const int per = (E + 31) / 32;
    const int b = min(lane * per, E), en = min(b + per, E);
    int sum = 0;
    for (int e = b; e < en; ++e) sum += pre_sh[e];
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    int acc = incl - sum;
    for (int e = b; e < en; ++e) {
      const int c = pre_sh[e];
      pre_sh[e] = acc;
      acc += c;
    }
  }
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_pairs) {
    const int e = topk_idx[i];
    if (e >= 0 && e < E) sorted_pair[pre_sh[e] + slot[i]] = i;
  }
  if (blockIdx.x == 0)
    moe_plan_body(counts_all, W, E, rank, send_row_base, src_pair_base, recv_expected, recv_base,
                  mblk_expert, n_mblocks, max_recv_rows, status, rows_sh, base_sh);
}

// Inverse of the slot map: sorted_pair[src_pair_base[e] + slot[i]] = i.
__global__ void moe_sort_pairs_kernel(const int* __restrict__ topk_idx, const int* __restrict__ slot,
                                      const int* __restrict__ src_pair_base, int n_pairs, int E,
                                      int* __restrict__ sorted_pair) {
  pdl_wait();                // chained with programmatic dependent launch: see prim/pdl.cuh
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  const int e = topk_idx[i];
  if (e < 0 || e >= E) return;
  sorted_pair[src_pair_base[e] + slot[i]] = i;
}

}  // namespace cb

using namespace cb;

extern "C" {

int cb_moe_router_topk(const void* logits, int T, int E, int K, void* topk_idx, void* topk_w,
                       void* stream) {
  if (E > 1024 || K > 32 || K < 1 || K > E) {
    set_last_error("router: E <= 1024 and 1 <= K <= min(32, E) required");
    return -1;
  }
  const int threads = 256;
  const int blocks = (T * 32 + threads - 1) / threads;
  router_topk_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(logits), T, E, K, static_cast<int*>(topk_idx),
      static_cast<float*>(topk_w));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Outputs must be zeroed by the caller (they are accumulated with atomics).
int cb_moe_dispatch_layout(const void* topk_idx, int T, int K, int R, int E, void* per_expert,
                           void* per_rank, void* in_rank, void* stream) {
  if (R < 1 || R > CB_MAX_RANKS || E % R != 0) {
    set_last_error("layout: 1 <= ranks <= 8 and experts divisible by ranks required");
    return -1;
  }
  dispatch_layout_kernel<<<(T + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(topk_idx), T, K, R, E, static_cast<int*>(per_expert),
      static_cast<int*>(per_rank), static_cast<unsigned char*>(in_rank));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int cb_moe_slots(const void* topk_idx, int n_pairs, int E, void* slot, void* counts, void* stream) {
  return launch_pdl(moe_slot_kernel, dim3(E), dim3(kSlotWarps * 32), 0,
                    static_cast<cudaStream_t>(stream), static_cast<const int*>(topk_idx), n_pairs,
                    E, static_cast<int*>(slot), static_cast<int*>(counts)) == cudaSuccess
             ? 0
             : -1;
}

int cb_moe_plan(const void* counts_all, int W, int E, int rank, void* send_row_base,
                void* src_pair_base, void* recv_expected, void* recv_base, void* mblk_expert,
                void* n_mblocks, int max_recv_rows, void* status, void* stream) {
  if (E > 1024 || E % W != 0) {
    set_last_error("plan: E <= 1024 and divisible by the world size required");
    return -1;
  }
  return launch_pdl(moe_plan_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const int*>(counts_all), W, E, rank,
                    static_cast<int*>(send_row_base), static_cast<int*>(src_pair_base),
                    static_cast<int*>(recv_expected), static_cast<int*>(recv_base),
                    static_cast<int*>(mblk_expert), static_cast<int*>(n_mblocks), max_recv_rows,
                    static_cast<uint32_t*>(status)) == cudaSuccess
             ? 0
             : -1;
}

// cb_moe_plan and cb_moe_sort_pairs as one launch.
int cb_moe_plan_sort(const void* counts_all, int W, int E, int rank, const void* topk_idx,
                     const void* slot, int n_pairs, void* sorted_pair, void* send_row_base,
                     void* src_pair_base, void* recv_expected, void* recv_base, void* mblk_expert,
                     void* n_mblocks, int max_recv_rows, void* status, void* stream) {
  if (E > 1024 || E % W != 0 || n_pairs < 1) {
    set_last_error("plan: E <= 1024 and divisible by the world size, at least one pair required");
    return -1;
  }
  return launch_pdl(moe_plan_sort_kernel, dim3((n_pairs + 255) / 256), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), static_cast<const int*>(counts_all), W, E,
                    rank, static_cast<const int*>(topk_idx), static_cast<const int*>(slot),
                    n_pairs, static_cast<int*>(sorted_pair), static_cast<int*>(send_row_base),
                    static_cast<int*>(src_pair_base), static_cast<int*>(recv_expected),
                    static_cast<int*>(recv_base), static_cast<int*>(mblk_expert),
                    static_cast<int*>(n_mblocks), max_recv_rows,
                    static_cast<uint32_t*>(status)) == cudaSuccess
             ? 0
             : -1;
}

int cb_moe_sort_pairs(const void* topk_idx, const void* slot, const void* src_pair_base,
                      int n_pairs, int E, void* sorted_pair, void* stream) {
  return launch_pdl(moe_sort_pairs_kernel, dim3((n_pairs + 255) / 256), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), static_cast<const int*>(topk_idx),
                    static_cast<const int*>(slot), static_cast<const int*>(src_pair_base), n_pairs,
                    E, static_cast<int*>(sorted_pair)) == cudaSuccess
             ? 0
             : -1;
}

}  // extern "C"
