// Programmatic dependent launch: a kernel launched with the attribute may start while its
// predecessor in the stream is still running; it must execute `pdl_wait()` before it touches
// anything the predecessor wrote (the wait returns once the predecessor has completed and its
// writes are visible).  `pdl_launch_dependents()` lets the NEXT kernel of the stream be
// scheduled from that point on, so its launch latency and prologue overlap this kernel.
//
// Every kernel of a chain calls pdl_wait() first thing, by every thread: a kernel that
// skipped it could let its own dependents start before its predecessors have finished.
//
// The reference chains its small expert-parallel kernels the same way
// (`cudaTriggerProgrammaticLaunchCompletion`: datasets/example079_deepep_jit_dispatch_notify/nv/
// empty_deepep_jit_dispatch_notify.cu:147; `cudaGridDependencySynchronize`:
// datasets/example081_deepep_jit_dispatch_copy_epilogue/nv/empty_deepep_jit_dispatch_copy_epilogue.cu:40;
// `kUsePDL`: datasets/example105_sglang_custom_allreduce_easy/empty_sglang_custom_allreduce_pull_easy.cu:105).
#pragma once
#include <cuda_runtime.h>

namespace cb {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Launch with programmatic stream serialisation allowed (the kernel must call pdl_wait()).
template <class... KArgs, class... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace cb
