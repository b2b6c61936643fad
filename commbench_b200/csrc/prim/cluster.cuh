// Thread-block-cluster helpers for CTA pairs (cluster of 2 along x).
//
// The reference's tensor-core GEMMs run as clusters of two CTAs that share one
// 256-row tile (`CLUSTER_SIZE = 2`, datasets/example051_thunderkitten_ag_gemm_easy/nv/
// empty_thunderkitten_ag_gemm.cu:73,152-238).  Here the pair talks through
// three things only: remote mbarrier arrivals, one remote 32-bit store (the
// abort word) and the cluster barrier at set-up and tear-down.  Operand tiles
// are never shared by a multicast load: each CTA fetches its own half.
#pragma once
#include "ptx.cuh"

namespace cb {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// shared::cta address of this CTA -> shared::cluster address of the same
// offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

// Execution + memory barrier over every thread of the cluster.  The unaligned
// forms are used: the callers arrive from diverged role code.
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  cluster_arrive();
  cluster_wait();
}

// One arrival on an mbarrier of any CTA of the cluster (shared::cluster address).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}

__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

}  // namespace cb
