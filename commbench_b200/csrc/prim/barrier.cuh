// Cross-GPU and grid-wide barriers; every spin is bounded and reports a status.
//
// Four designs, matching what the reference's examples use:
//  * rank_barrier_block  - epoch flag matrix, one word per (channel, source rank);
//                          all-pairs signal + wait like the relaxedSignal/wait mesh of
//                          datasets/example040_mscclpp_relaxedsingal_easy/
//                          empty_mscclpp_relaxedsingal_easy.cu:1-21, made monotonic so no reset
//                          pass is needed.
//  * addsub_barrier_warp - the self-resetting add/sub matrix barrier of
//                          datasets/example017_intranode_gpu_barrier/nv/
//                          empty_intranode_gpu_barrier.cu:38-53.
//  * nvls_barrier_block  - one multimem.red on the multicast alias of the pads
//                          (datasets/example048_thunderkitten_all_reduce_easy/nv/
//                          empty_thunderkitten_all_reduce.cu:96-115).
//  * grid_barrier        - counter barrier among the CTAs of one launch (the DeviceSyncer of
//                          datasets/example031_msclpp_allreduce_rsag_zero_easy/
//                          empty_mscclpp_allreduce_easy.cu:85); needs a co-resident grid.
#pragma once
#include "comm.h"
#include "ptx.cuh"

namespace cb {

// Phase identifiers recorded in status words.
enum : uint32_t {
  PH_BARRIER_START = 1,
  PH_BARRIER_MID = 2,
  PH_BARRIER_END = 3,
  PH_NVLS_BARRIER = 4,
  PH_GRID_BARRIER = 5,
  PH_ADDSUB_BARRIER = 6,
};

// All threads of the CTA call this.  Orders every global write the CTA made
// before the call ahead of the peers' reads after their matching call.
// `value` must be the same on every rank for the same barrier instance and grow
// by one per instance on the channel.
__device__ __forceinline__ bool rank_barrier_block(const CbComm& c, uint32_t ch, uint32_t value,
                                                   uint32_t phase) {
  __syncthreads();
  bool ok = true;
  if (threadIdx.x < static_cast<uint32_t>(c.world)) {
    const uint32_t peer = threadIdx.x;
    st_release_sys(c.pad[peer] + ch * CB_MAX_RANKS + c.rank, value);
    ok = wait_flag_ge_sys(c.pad[c.rank] + ch * CB_MAX_RANKS + peer, value, c.timeout_ns, c.status,
                          phase, peer);
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Signal only (no wait): "my data for this channel is ready / I am done with yours".
__device__ __forceinline__ void rank_signal_block(const CbComm& c, uint32_t ch, uint32_t value) {
  __syncthreads();
  if (threadIdx.x < static_cast<uint32_t>(c.world)) {
    st_release_sys(c.pad[threadIdx.x] + ch * CB_MAX_RANKS + c.rank, value);
  }
}
__device__ __forceinline__ bool rank_wait_block(const CbComm& c, uint32_t ch, uint32_t value,
                                                uint32_t phase) {
  bool ok = true;
  if (threadIdx.x < static_cast<uint32_t>(c.world)) {
    ok = wait_flag_ge_sys(c.pad[c.rank] + ch * CB_MAX_RANKS + threadIdx.x, value, c.timeout_ns,
                          c.status, phase, threadIdx.x);
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// One multimem.red bumps counter `ch` on every rank; wait until all `world`
// ranks did so for this instance.  `value` counts instances (1, 2, ...).
__device__ __forceinline__ bool nvls_barrier_block(const CbComm& c, uint32_t ch, uint32_t value) {
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) {
    uint32_t* mc = c.mc_pad + CB_PAD_NVLS_BASE + ch;
    asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(1u)
                 : "memory");
    ok = wait_flag_ge_sys(c.pad[c.rank] + CB_PAD_NVLS_BASE + ch,
                          value * static_cast<uint32_t>(c.world), c.timeout_ns, c.status,
                          PH_NVLS_BARRIER, ch);
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Self-resetting barrier on an N x N int matrix per rank: add 1 to my own row
// entry for each peer, subtract 1 from the peer's row entry for me, spin until my
// row is back to <= 0.  One warp per GPU (lane = peer).
__device__ __forceinline__ bool addsub_barrier_warp(int* const* rows /*[world] peer-mapped*/,
                                                    int rank, int world, uint64_t timeout_ns,
                                                    uint32_t* status) {
  const uint32_t lane = lane_id();
  __threadfence_system();
  bool ok = true;
  if (lane < static_cast<uint32_t>(world)) {
    atomicAdd_system(rows[rank] + rank * world + lane, 1);
    atomicSub_system(rows[lane] + lane * world + rank, 1);
  }
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 0;; ++it) {
    int v = 0;
    if (lane < static_cast<uint32_t>(world)) {
      v = *reinterpret_cast<volatile int*>(rows[rank] + rank * world + lane);
    }
    if (__ballot_sync(0xffffffffu, v > 0) == 0u) break;
    if ((it & 63u) == 63u && globaltimer_ns() - t0 > timeout_ns) {
      ok = false;
      break;
    }
  }
  if (!ok && lane == 0) report_status(status, CB_TIMEOUT_PEER_FLAG, PH_ADDSUB_BARRIER, 0);
  __threadfence_system();
  return ok;
}

// Barrier among the CTAs of ONE launch (all must be resident).  `counter` is a
// zero-initialised word that keeps counting up; `generation` is the number of
// barriers this launch has completed on it before this call.
__device__ __forceinline__ bool grid_barrier(uint32_t* counter, uint32_t base, uint32_t generation,
                                             uint32_t nblocks, uint64_t timeout_ns,
                                             uint32_t* status) {
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) {
    red_release_gpu_add(counter, 1u);
    ok = wait_flag_ge_gpu(counter, base + (generation + 1u) * nblocks, timeout_ns, status,
                          PH_GRID_BARRIER, generation);
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

}  // namespace cb
