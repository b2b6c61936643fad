// Pieces shared by the fused GEMM+collective kernels.
//
// Synchronisation scheme (no cross-GPU barrier on the hot path):
//  * every op instance owns a local call counter `seq`; buffers and flags in
//    symmetric memory exist twice and call k uses copy k&1;
//  * a rank can only be two calls ahead of a peer after that peer has finished
//    the older call (each call of these ops needs data from every peer), so
//    copy k&1 is never overwritten while call k still reads it;
//  * flags count arrivals and are zeroed by their consumer right after use, so
//    nothing depends on the shapes of earlier calls;
//  * the last CTA to leave bumps `seq` (all CTAs read it first thing).
#pragma once
#include "../gemm/gemm_sm100.cuh"
#include "../prim/barrier.cuh"
#include "../prim/multimem.cuh"

namespace cb {

enum : uint32_t {
  PH_AG_ROWS = 32,     // waiting for a peer's A row block (detail = row block)
  PH_RS_TILE = 33,     // waiting for partial tiles of an output tile (detail = tile)
  PH_AR_TILE = 34,     // same, all-reduce
  PH_AR_DONE = 35,     // waiting for the reduced tiles from their owners
  PH_COMM_LOAD = 36,   // comm worker waiting for its own bulk load
};

struct FusedSeq {
  uint32_t* seq;        // call counter (local device memory)
  uint32_t* done_ctas;  // CTAs that left the current call
};

// All threads call it first thing; returns the call's parity.
__device__ __forceinline__ uint32_t fused_begin(const FusedSeq& s) {
  return ld_volatile(s.seq) & 1u;
}
// All threads call it last thing.  `nctas` = CTAs of this (virtual) rank.
__device__ __forceinline__ void fused_end(const FusedSeq& s, uint32_t nctas) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(s.done_ctas, 1u);
    if (prev == nctas - 1u) {
      *s.done_ctas = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(s.seq) = ld_volatile(s.seq) + 1u;
    }
  }
}

// Sum `nsrc` bf16 vectors (8 values each) in fp32.
__device__ __forceinline__ uint4 sum_bf16x8(const uint4* v, int nsrc) {
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  for (int s = 0; s < nsrc; ++s) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[s]);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 t = __bfloat1622float2(h[k]);
      acc[2 * k] += t.x;
      acc[2 * k + 1] += t.y;
    }
  }
  uint4 r;
  __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int k = 0; k < 4; ++k) o[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
  return r;
}

template <int W>
__device__ __forceinline__ uint4 sum_bf16x8_t(const uint4 (&v)[W]) {
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
  for (int s = 0; s < W; ++s) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[s]);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 t = __bfloat1622float2(h[k]);
      acc[2 * k] += t.x;
      acc[2 * k + 1] += t.y;
    }
  }
  uint4 r;
  __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int k = 0; k < 4; ++k) o[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
  return r;
}

// Sum of W staged copies of one [ROWS x VPR vectors] tile, many loads in flight
// per thread (L2-coherent loads: the copies were written by peers).
//   src(s, v)  -> address of vector v of copy s          (callable)
//   dst(v, x)  -> consumes the reduced vector            (callable)
//   valid(v)   -> false for vectors outside the tensor   (callable)
template <int W, int NVEC, class Src, class Dst, class Valid>
__device__ __forceinline__ void reduce_tile_copies(Src src, Dst dst, Valid valid) {
  constexpr int U = W >= 8 ? 2 : (W >= 4 ? 4 : 8);
  for (int v0 = threadIdx.x; v0 < NVEC; v0 += blockDim.x * U) {
    uint4 parts[U][W];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * static_cast<int>(blockDim.x);
      ok[u] = v < NVEC && valid(v);
      if (ok[u]) {
#pragma unroll
        for (int s = 0; s < W; ++s) parts[u][s] = __ldcg(src(s, v));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (ok[u]) dst(v0 + u * static_cast<int>(blockDim.x), sum_bf16x8_t<W>(parts[u]));
    }
  }
}

}  // namespace cb
