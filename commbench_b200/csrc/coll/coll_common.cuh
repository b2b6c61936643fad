// Shared pieces of the collective kernels: the argument block, the rank
// emulation hook, dtype-generic 16-byte vector arithmetic.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../prim/barrier.cuh"
#include "../prim/multimem.cuh"

namespace cb {

enum CbDtype : int { CB_BF16 = 0, CB_F16 = 1, CB_F32 = 2 };

// One argument block per (virtual) rank.  `sym[r]` is rank r's copy of the
// symmetric buffer the op works through (peer-mapped; sym[rank] is local);
// `mc` is its multicast alias or nullptr.  `in`/`out` are ordinary local tensors
// (they may alias sym[rank] when the caller already works in symmetric memory).
struct CollArgs {
  CbComm comm;
  void* sym[CB_MAX_RANKS];
  void* mc;
  const void* in;
  void* out;
  unsigned long long nbytes;  // bytes of the logical message (per-op meaning documented there)
  int copy_in;                // 1: kernel first copies `in` into sym[rank]
  int copy_out;               // 1: result is taken from sym[rank] into `out` at the end
  int root;                   // broadcast root
  int dtype;
  // 4-D all-to-all geometry (elements): [B, S_local, H, D] <-> [B, S, H_local, D]
  int a2a_b, a2a_s_local, a2a_h, a2a_d, a2a_to_heads;
  // Tuning: 16-byte vectors each thread keeps in flight in the bandwidth loops (0: the
  // kernel's default of 4; values are rounded down to 2, 4 or 8).
  int unroll;
  // Bit 0 picks the push form where an op has one: two-shot all-reduce stores each reduced
  // vector to every rank instead of letting the ranks pull it in a second phase; flat
  // all-to-all stores chunk p of `in` into rank p's sym[] instead of pulling.
  int variant;
};

// Several ranks can be emulated inside ONE launch on one GPU: the grid gets
// `world` slices along y and slice y uses emu[y].  This exercises the same
// device code (flags, peers, barriers) without two kernels that wait on each
// other ever running as separate launches.  Such launches are cooperative so
// that all slices are resident together.
__device__ __forceinline__ const CollArgs& pick_args(const CollArgs& a, const CollArgs* emu) {
  return emu != nullptr ? emu[blockIdx.y] : a;
}

// Channel of this CTA on the signal pad: unique per (virtual rank's) CTA.
__device__ __forceinline__ uint32_t cta_channel(uint32_t base) { return base + blockIdx.x; }

template <int DT>
struct Vec16;  // 16-byte vector arithmetic in fp32

template <>
struct Vec16<CB_BF16> {
  static constexpr int N = 8;
  __device__ static void unpack(uint4 v, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ static uint4 pack(const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
  }
  __device__ static uint4 mm_reduce(const void* mc) { return mm_ld_reduce_bf16x8(mc); }
};
template <>
struct Vec16<CB_F16> {
  static constexpr int N = 8;
  __device__ static void unpack(uint4 v, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ static uint4 pack(const float (&f)[8]) {
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return v;
  }
  __device__ static uint4 mm_reduce(const void* mc) { return mm_ld_reduce_f16x8(mc); }
};
template <>
struct Vec16<CB_F32> {
  static constexpr int N = 4;
  __device__ static void unpack(uint4 v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  __device__ static uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
  __device__ static uint4 mm_reduce(const void* mc) {
    float4 t = mm_ld_reduce_f32x4(mc);
    return make_uint4(__float_as_uint(t.x), __float_as_uint(t.y), __float_as_uint(t.z),
                      __float_as_uint(t.w));
  }
};

// [begin, end) of slice `i` of `n` items cut into `parts` nearly equal slices.
__device__ __forceinline__ void slice_of(unsigned long long n, uint32_t parts, uint32_t i,
                                         unsigned long long* begin, unsigned long long* end) {
  const unsigned long long per = (n + parts - 1) / parts;
  unsigned long long b = per * i;
  unsigned long long e = b + per;
  if (b > n) b = n;
  if (e > n) e = n;
  *begin = b;
  *end = e;
}

}  // namespace cb
