// NVLS (NVSwitch multicast) instructions on a multicast address: one load that
// returns the sum over every GPU's copy, one store that lands on every GPU.
//
// Same instructions the reference uses through ThunderKittens
// (datasets/example048_thunderkitten_all_reduce_easy/nv/
// empty_thunderkitten_all_reduce.cu:64-94) and through the NCCL device API's
// ncclMultimemReduceSumCopy (datasets/example043_nccl_device_api_intranode_allreduce/
// empty_nccl_device_api_allreduce.cu:50-62).
#pragma once
#include "ptx.cuh"

namespace cb {

// 8 bf16 values (16 B) summed across all ranks, fp32 accumulation in the switch.
__device__ __forceinline__ uint4 mm_ld_reduce_bf16x8(const void* mc_ptr) {
  uint4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc_ptr)
      : "memory");
  return v;
}
__device__ __forceinline__ uint4 mm_ld_reduce_f16x8(const void* mc_ptr) {
  uint4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc_ptr)
      : "memory");
  return v;
}
__device__ __forceinline__ float4 mm_ld_reduce_f32x4(const void* mc_ptr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}
// 16-byte store replicated to every rank bound to the multicast object.
__device__ __forceinline__ void mm_st_v4(void* mc_ptr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_ptr),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void mm_red_add_relaxed_u32(uint32_t* mc_ptr, uint32_t v) {
  asm volatile("multimem.red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(mc_ptr), "r"(v)
               : "memory");
}
__device__ __forceinline__ void mm_red_add_u32(uint32_t* mc_ptr, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_ptr), "r"(v)
               : "memory");
}

}  // namespace cb
