// The context-parallel attention kernel (fa_cp.cuh) and its launch helper.
#include "cp_launch.h"
#include "fa_cp.cuh"

#include <string>

#include "../symm/driver_api.h"

namespace cb {

int cp_num_items(const FaCpParams& p) {
  int pairs = 0;
  for (int i = 0; i < p.nqseg; ++i) pairs += (p.qseg[i].nrows + 2 * CP_BM - 1) / (2 * CP_BM);
  return pairs * p.heads * p.B;
}

int cp_launch(const FaCpParams& p, int grid, cudaStream_t st) {
  static bool attr_set = false;
  cudaError_t e = cudaSuccess;
  if (!attr_set) {
    e = cudaFuncSetAttribute(fa_cp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, CP_SMEM);
    if (e != cudaSuccess) {
      set_last_error(std::string("cudaFuncSetAttribute(fa_cp): ") + cudaGetErrorString(e));
      return -1;
    }
    attr_set = true;
  }
  if (grid < 1) return 0;
  fa_cp_kernel<<<grid, CP_THREADS, CP_SMEM, st>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(std::string("context-parallel attention launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // namespace cb
