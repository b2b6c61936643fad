// Thin inline-PTX wrappers: scoped loads/stores/reductions on flag words,
// fences, timers, warp election.  Everything here is plain sm_100a PTX.
//
// Covers the flag primitives that the reference spreads over its examples:
// ld.acquire.sys / red.release.sys ping-pong flags
// (datasets/example073_GPU_p2p_pingpong_latency/nv/empty_p2p_pingpong_latency.cu:30-43),
// st.volatile pushes (datasets/example101_sglang_qknorm_fused_easy/
// empty_sglang_qknorm_fused_easy.cu:147-161) and %globaltimer / nanosleep
// (datasets/example076_GPU_globaltimer_nanosleep/nv/empty_globaltimer_nanosleep.cu:25-36).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "status.h"

namespace cb {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t l;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
  return l;
}

__device__ __forceinline__ uint32_t smid() {
  uint32_t s;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(s));
  return s;
}

// One lane of a fully converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- flag words
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_volatile(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_volatile_v2f(float2* p, float2 v) {
  asm volatile("st.volatile.global.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(v.x), "f"(v.y)
               : "memory");
}
__device__ __forceinline__ float2 ld_volatile_v2f(const float2* p) {
  float2 v;
  asm volatile("ld.volatile.global.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t atom_add_acqrel_sys(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.sys.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v)
               : "memory");
  return old;
}
__device__ __forceinline__ uint64_t atom_add_relaxed_sys_u64(uint64_t* p, uint64_t v) {
  uint64_t old;
  asm volatile("atom.relaxed.sys.global.add.u64 %0, [%1], %2;" : "=l"(old) : "l"(p), "l"(v)
               : "memory");
  return old;
}
__device__ __forceinline__ void fence_acq_rel_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}
__device__ __forceinline__ void fence_acq_rel_gpu() {
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
}
// Orders generic-proxy accesses with async-proxy (TMA / tcgen05) accesses.
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------ 16-byte access
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Peer / freshly written data: no non-coherent path, relaxed at system scope.
__device__ __forceinline__ uint4 ld_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_v4(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_sys_v4(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// ---------------------------------------------------------------- error word
// First error wins; later ones are dropped so the host sees the root cause.
__device__ __forceinline__ void report_status(uint32_t* status, uint32_t code, uint32_t phase,
                                              uint32_t detail) {
  if (status != nullptr) {
    atomicCAS(status, 0u, (code << 24) | ((phase & 0xffu) << 16) | (detail & 0xffffu));
    fence_acq_rel_sys();
  }
}

// Bounded wait until *flag >= target (wrap-safe).  Returns false on time-out,
// after recording the status word.  `timeout_ns` is a %globaltimer budget; the
// iteration cap is a second guard in case the timer misbehaves.
//
// Keep the number of threads that poll one remotely-updated word small (a handful): with
// every CTA of a grid polling the same word, the peers' atomics to it - and everything
// queued behind them on the link - were held up for hundreds of microseconds.  Where a
// whole grid must wait for one remote event, one CTA polls it and republishes it in a
// local word for the others (see the fused GEMM + all-reduce kernel).
__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool wait_flag_ge_sys(const uint32_t* flag, uint32_t target,
                                                 uint64_t timeout_ns, uint32_t* status,
                                                 uint32_t phase, uint32_t detail) {
  if (static_cast<int32_t>(ld_acquire_sys(flag) - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 0; it < 0x7fffffffu; ++it) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - target) >= 0) return true;
    if ((it & 63u) == 63u) {
      if (globaltimer_ns() - t0 > timeout_ns) break;
      if (status != nullptr && ld_volatile(status) != 0u) break;  // somebody already failed
    }
    // A few back-to-back polls for the latency-bound case, then paced ones: system-scope
    // polls from a whole grid of waiting CTAs measurably delay the peers' stores into this
    // GPU (see the paced variant below), and the CTAs that finish a bandwidth loop first
    // wait here while the others' data is still arriving.
    if (it >= 16u) __nanosleep(it < 64u ? 128u : (it < 256u ? 512u : 1024u));
  }
  report_status(status, CB_TIMEOUT_PEER_FLAG, phase, detail);
  return false;
}

// Paced variant for waits that many CTAs of a grid sit in at the same time (one per tile,
// per expert, ...): acquire polls `poll_ns` apart (an acquire load per poll measured cheaper
// than relaxed polls plus a system fence at the end).  Measured on B200: ~100 SMs polling back to back delayed the peers' stores and
// atomics into this GPU by 100-400 us; a few hundred nanoseconds between polls removed it.
__device__ __forceinline__ bool wait_flag_ge_sys_paced(const uint32_t* flag, uint32_t target,
                                                       uint64_t timeout_ns, uint32_t* status,
                                                       uint32_t phase, uint32_t detail,
                                                       uint32_t poll_ns) {
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 0; it < 0x7fffffffu; ++it) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - target) >= 0) return true;
    if ((it & 15u) == 15u) {
      if (globaltimer_ns() - t0 > timeout_ns) break;
      if (status != nullptr && ld_volatile(status) != 0u) break;
    }
    if (poll_ns > 0u) __nanosleep(poll_ns);
  }
  report_status(status, CB_TIMEOUT_PEER_FLAG, phase, detail);
  return false;
}
constexpr uint32_t kPacedPollNs = 300u;

__device__ __forceinline__ bool wait_flag_ge_gpu(const uint32_t* flag, uint32_t target,
                                                 uint64_t timeout_ns, uint32_t* status,
                                                 uint32_t phase, uint32_t detail) {
  if (static_cast<int32_t>(ld_relaxed_gpu(flag) - target) >= 0) {
    fence_acq_rel_gpu();
    return true;
  }
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 0; it < 0x7fffffffu; ++it) {
    if (static_cast<int32_t>(ld_relaxed_gpu(flag) - target) >= 0) {
      fence_acq_rel_gpu();
      return true;
    }
    if ((it & 63u) == 63u) {
      if (globaltimer_ns() - t0 > timeout_ns) break;
      if (status != nullptr && ld_volatile(status) != 0u) break;
    }
    if (it > 32u) __nanosleep(32);
  }
  report_status(status, CB_TIMEOUT_LOCAL_FLAG, phase, detail);
  return false;
}

}  // namespace cb
