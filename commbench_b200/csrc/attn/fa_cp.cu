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

static int g_cp_poly = 0;

template <int kPoly>
static int cp_launch_t(const FaCpParams& p, int grid, cudaStream_t st) {
  static bool attr_set = false;
  cudaError_t e = cudaSuccess;
  if (!attr_set) {
    e = cudaFuncSetAttribute(fa_cp_kernel<kPoly>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             CP_SMEM);
    if (e != cudaSuccess) {
      set_last_error(std::string("cudaFuncSetAttribute(fa_cp): ") + cudaGetErrorString(e));
      return -1;
    }
    attr_set = true;
  }
  fa_cp_kernel<kPoly><<<grid, CP_THREADS, CP_SMEM, st>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(std::string("context-parallel attention launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

int cp_launch(const FaCpParams& p, int grid, cudaStream_t st) {
  if (grid < 1) return 0;
  switch (g_cp_poly) {
    case 2: return cp_launch_t<2>(p, grid, st);
    case 3: return cp_launch_t<3>(p, grid, st);
    case 4: return cp_launch_t<4>(p, grid, st);
    default: return cp_launch_t<0>(p, grid, st);
  }
}

}  // namespace cb

using namespace cb;

extern "C" {

// Every n-th pair of keys computes its exponential on the FMA pipe (0 = none, 2, 3 or 4).
void cb_attn_set_poly_every(int n) { g_cp_poly = n; }

// Local attention over one key/value chunk: q [B, Sq, Hq, 128], k/v [B, Skv, Hkv, 128],
// o [B, Sq, Hq, 128] bf16 contiguous; lse [B, Hq, Sq] fp32.  q_offset / kv_offset are the global
// sequence positions of the first query / key; with `causal`, key j is visible to query i iff
// kv_offset + j <= q_offset + i.  One key segment, one query segment, no communication CTAs.
int cb_attn_fwd4(const void* q, const void* k, const void* v, void* o, void* lse, int B, int Sq,
                 int Skv, int Hq, int Hkv, int q_offset, int kv_offset, int causal, float scale,
                 void* status, void* stream) {
  if (B < 1 || Sq < 1 || Skv < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0) {
    set_last_error("attention: bad shape (Hq must be a multiple of Hkv)");
    return -1;
  }
  FaCpParams p = {};
  if (cb_attn_make_tmap_bshd(&p.tm_q_local, q, B * Sq, Hq)) return -1;
  if (cb_attn_make_tmap_bshd(&p.tm_k, k, B * Skv, Hkv)) return -1;
  if (cb_attn_make_tmap_bshd(&p.tm_v, v, B * Skv, Hkv)) return -1;
  p.nseg = 1;
  p.seg[0].row0 = 0;
  p.seg[0].kpos0 = kv_offset;
  p.seg[0].nkeys = Skv;
  p.seg[0].flag = -1;
  p.nqseg = 1;
  p.qseg[0].map = -1;
  p.qseg[0].row0 = 0;
  p.qseg[0].qpos0 = q_offset;
  p.qseg[0].nrows = Sq;
  p.qseg[0].out = 0;
  p.o[0] = static_cast<__nv_bfloat16*>(o);
  p.lse[0] = static_cast<float*>(lse);
  p.o_rows[0] = Sq;
  p.B = B;
  p.heads = Hq;
  p.o_heads = Hq;
  p.kv_group = Hq / Hkv;
  p.q_bstride = Sq;
  p.kv_bstride = Skv;
  p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = static_cast<uint32_t*>(status);
  p.timeout_ns = 2000000000ull;
  return cp_launch(p, cp_num_items(p), static_cast<cudaStream_t>(stream));
}

}  // extern "C"
