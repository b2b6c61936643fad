// TMA (cp.async.bulk / cp.async.bulk.tensor) wrappers.  No load here carries a
// cluster-multicast qualifier: every CTA fetches its own tiles, and tiles that
// come from another GPU are first pushed into local memory by their owner.
//
// 1-D bulk loads mirror datasets/example094_TMA_bulk_copy_gmem_to_smem/nv/
// empty_tma_bulk_copy.cu:28-58; tensor-map loads/stores are what the reference's
// ThunderKittens examples obtain from `tma::load_async / store_async`
// (datasets/example046_thunderkitten_all_gather_easy/nv/
// empty_thunderkitten_all_gather.cu:56-104).
//
// Alignment rules enforced by the host wrappers that build the coordinates:
// the innermost coordinate times the element size is a multiple of 16 bytes,
// shared-memory tiles are 128-byte aligned (1024 for 128B swizzle).
#pragma once
#include <cuda.h>

#include "mbarrier.cuh"

namespace cb {

// ------------------------------------------------------------------ 1-D bulk
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                             uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_store_1d(void* gmem_dst, const void* smem_src,
                                              uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Source smem may be reused once the reads are done.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Writes of the groups have been performed (needed before signalling a consumer).
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// --------------------------------------------------------------- tensor maps
__device__ __forceinline__ void tmap_prefetch(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// Same, with shared-memory addresses already converted.
__device__ __forceinline__ void tma_load_2d_addr(uint32_t smem_dst, const CUtensorMap* m, int x,
                                                 int y, uint32_t bar_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar_addr)
      : "memory");
}
// CTA-pair form: the data lands in THIS CTA's shared memory, the completion
// bytes are counted on an mbarrier that may live in the partner CTA
// (`bar_cluster_addr` is a shared::cluster address).  Not a multicast load.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* m, int x,
                                                 int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, int x, int y,
                                            int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x,
                                             int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
          reinterpret_cast<uint64_t>(m)),
      "r"(x), "r"(y), "r"(smem_u32(smem_src))
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* smem_src, int x,
                                             int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(
          reinterpret_cast<uint64_t>(m)),
      "r"(x), "r"(y), "r"(z), "r"(smem_u32(smem_src))
      : "memory");
}
// Element-wise add into global memory (bf16 / f32 maps); used for in-flight reductions.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, const void* smem_src,
                                                  int x, int y) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], "
      "[%3];" ::"l"(reinterpret_cast<uint64_t>(m)),
      "r"(x), "r"(y), "r"(smem_u32(smem_src))
      : "memory");
}

}  // namespace cb
