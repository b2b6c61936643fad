// Kernel launch helper for the tcgen05 GEMM kernels: plain, as clusters of two
// CTAs (CTA pairs), and / or cooperative (rank emulation, where the CTAs of the
// virtual ranks wait on one another and must be co-resident).
//
// The reference launches its cluster kernels the same way (`cudaLaunchKernelEx`
// with a cluster dimension and a dynamic shared-memory attribute:
// datasets/example051_thunderkitten_ag_gemm_easy/nv/empty_thunderkitten_ag_gemm.cu:271-308).
#pragma once
#include <cuda_runtime.h>

namespace cb {

template <class... KArgs, class... Args>
inline cudaError_t launch_gemm_kernel(void (*kernel)(KArgs...), int grid, int threads, int smem,
                                      cudaStream_t st, int cluster, bool cooperative,
                                      Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(static_cast<unsigned>(threads));
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = static_cast<unsigned>(cluster);
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (cooperative) {
    attr[n].id = cudaLaunchAttributeCooperative;
    attr[n].val.cooperative = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace cb
