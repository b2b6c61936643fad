// Dispatch push (fp8 quantisation fused into the send), dequantising receive,
// SwiGLU and the weighted combine reduction.  See moe_kernels.cu for the overall
// design and the reference counterparts.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../prim/barrier.cuh"
#include "../prim/pdl.cuh"

namespace cb {
void set_last_error(const std::string& s);

enum : uint32_t { PH_MOE_ARRIVE2 = 48, PH_MOE_COMBINE2 = 49 };

struct MoeSendArgs {
  const __nv_bfloat16* x;     // [T, H] this rank's tokens
  const int* topk_idx;        // [T*K]
  const float* topk_w;        // [T*K]
  const int* sorted_pair;     // [T*K] pairs in expert-major order
  const int* src_pair_base;   // [E]
  const int* my_counts;       // [E] selections of each expert among my tokens
  const int* send_row_base;   // [E] first destination row
  uint8_t* recv_x[CB_MAX_RANKS];      // fp8 [max_rows, H] on each rank
  float* recv_scale[CB_MAX_RANKS];    // [max_rows, H/128]
  int2* recv_meta[CB_MAX_RANKS];      // [max_rows] {source rank, source pair index}
  uint32_t* arrived[CB_MAX_RANKS];    // [E/W] rows arrived per local expert
  int rank, world, T, K, H, E, max_rows;
  uint32_t* status;
  int per_token;              // 1: one copy of a token per destination RANK (see the kernel)
};

// grid (E, slices).  Warp per row: load the token's bf16 row, per-128-channel
// absmax -> scale, quantise to e4m3, write 8 bytes per lane to the destination
// row; the CTA then releases once and bumps the expert's arrival counter.
//
// per_token = 0 (expanded layout): every (token, expert) selection carries its own copy of the
// token, written at its final row of the destination's per-expert receive buffer.
// per_token = 1: a token crosses NVLink once per destination RANK, however many of that rank's
// experts it selected (the non-expanded mode of the reference's dispatch,
// datasets/example081_deepep_jit_dispatch_copy_epilogue/nv/
// empty_deepep_jit_dispatch_copy_epilogue.cu:11,49-58: `kDoExpand`).  The copy goes to row
// rank * T + token of the destination's buffer - a position both sides can compute, so no
// second count exchange is needed - sent by the first of the token's selections that lives on
// that rank; every selection still writes its {source rank, pair} word at its final row, and the
// receive kernel expands from there.
__global__ void __launch_bounds__(256)
    moe_dispatch_send_kernel(const __grid_constant__ MoeSendArgs a) {
  pdl_wait();                // chained with programmatic dependent launch: see prim/pdl.cuh
  pdl_launch_dependents();
  const int e = blockIdx.x;
  const int El = a.E / a.world;
  const int dst = e / El;
  const int cnt = a.my_counts[e];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int nvec = a.H / 8;        // 16-byte vectors per row
  const int groups = a.H / 128;
  int handled = 0;
  for (int r = blockIdx.y * warps + warp; r < cnt; r += gridDim.y * warps) {
    const int pair = a.sorted_pair[a.src_pair_base[e] + r];
    const int token = pair / a.K;
    const long long row = static_cast<long long>(a.send_row_base[e]) + r;
    if (row >= a.max_rows) continue;  // plan kernel already reported the overflow
    long long drow = row;
    bool send = true;                 // the same for every lane: `pair` belongs to the warp
    if (a.per_token) {
      const int k = pair - token * a.K;
      const int lo = dst * El, hi = lo + El;
      for (int kk = 0; kk < k; ++kk) {
        const int ee = a.topk_idx[token * a.K + kk];
        if (ee >= lo && ee < hi) send = false;     // an earlier selection already sends the token
      }
      drow = static_cast<long long>(a.rank) * a.T + token;
    }
    const uint4* __restrict__ src =
        reinterpret_cast<const uint4*>(a.x + static_cast<size_t>(token) * a.H);
    uint2* __restrict__ dq = reinterpret_cast<uint2*>(a.recv_x[dst] + drow * a.H);
    float* __restrict__ ds = a.recv_scale[dst] + drow * groups;
    // H is a multiple of 256, so every lane makes the same number of trips (the shuffles below
    // need the whole warp); four rows of loads in flight per lane.
#pragma unroll 4
    for (int v = lane; send && v < nvec; v += 32) {
      const uint4 raw = src[v];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      float f[8];
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
        amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
      }
      // 16 lanes share one 128-channel group
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float scale = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
      const float inv = 1.0f / scale;
      uint32_t w[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
            make_float2(f[4 * i] * inv, f[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
            make_float2(f[4 * i + 2] * inv, f[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
        w[i] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
      }
      dq[v] = make_uint2(w[0], w[1]);
      if ((lane & 15) == 0) ds[v / 16] = scale;
    }
    if (lane == 0) a.recv_meta[dst][row] = make_int2(a.rank, pair);
    ++handled;
  }
  // CTA-wide count of rows written, one release, one counter bump.
  __shared__ int total;
  if (threadIdx.x == 0) total = 0;
  __syncthreads();
  if (lane == 0 && handled > 0) atomicAdd(&total, handled);
  __syncthreads();
  if (threadIdx.x == 0 && total > 0) {
    fence_acq_rel_sys();
    red_relaxed_sys_add(a.arrived[dst] + (e - dst * El), static_cast<uint32_t>(total));
  }
}

struct MoeRecvArgs {
  const uint8_t* recv_x;      // fp8 [max_rows, H]
  const float* recv_scale;    // [max_rows, H/128]
  int2* recv_meta;            // [max_rows]
  __nv_bfloat16* a_out;       // bf16 [max_rows, H]  (grouped-GEMM input)
  uint32_t* arrived;          // [El]
  const int* recv_expected;   // [El]
  const int* recv_base;       // [El+1]
  int H, max_rows;
  unsigned long long timeout_ns;
  uint32_t* status;
  uint32_t* ctas_done;        // [El] zero-initialised words of this rank, or null (see the kernel)
  int per_token;              // 1: rows were sent once per token and rank; expand them here
  int T, K;                   // tokens per rank and selections per token (per_token only)
  int stage_rows;             // rows of recv_x / recv_scale (per_token only: world * T)
};

// grid (El, slices).  Waits until the expert's rows are all in, then
// dequantises them to bf16; padding rows (up to the next multiple of 128) are
// zeroed and marked with source rank -1 so later stages skip them.
// With `ctas_done` set, the last CTA of an expert to finish clears that expert's arrival
// counter, so no separate fill launch is needed between two calls.  This is early enough: a peer
// cannot send rows of its NEXT call before it has this rank's combine rows of the current one,
// and those leave after this kernel in stream order.
__global__ void __launch_bounds__(256)
    moe_recv_dequant_kernel(const __grid_constant__ MoeRecvArgs a) {
  pdl_wait();                // chained with programmatic dependent launch: see prim/pdl.cuh
  pdl_launch_dependents();
  const int j = blockIdx.x;
  const int expect = a.recv_expected[j];
  const int base = a.recv_base[j];
  const int padded = a.recv_base[j + 1] - base;
  bool ok = true;
  if (a.per_token) {
    // A row of this expert may have been sent on behalf of another expert of this rank (the
    // token's first selection here), so every counter of the rank has to be complete.  One
    // thread polls them one after the other (starting at its own): all must be complete
    // anyway, and few pollers leave the memory system to the rows still arriving.
    if (threadIdx.x == 0) {
      const int n = static_cast<int>(gridDim.x);
      for (int t = 0; t < n && ok; ++t) {
        const int i = (j + t) % n;
        const int ex = a.recv_expected[i];
        if (ex > 0)
          ok = wait_flag_ge_sys(a.arrived + i, static_cast<uint32_t>(ex), a.timeout_ns, a.status,
                                PH_MOE_ARRIVE2, i);
      }
    }
  } else if (threadIdx.x == 0 && expect > 0) {
    ok = wait_flag_ge_sys(a.arrived + j, static_cast<uint32_t>(expect), a.timeout_ns, a.status,
                          PH_MOE_ARRIVE2, j);
  }
  const bool all_ok = __syncthreads_and(ok ? 1 : 0) != 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int nvec = a.H / 8;
  const int groups = a.H / 128;
  for (int r = blockIdx.y * warps + warp; all_ok && r < padded; r += gridDim.y * warps) {
    const long long row = static_cast<long long>(base) + r;
    if (row >= a.max_rows) continue;
    uint4* __restrict__ out = reinterpret_cast<uint4*>(a.a_out + row * a.H);
    if (r >= expect) {
      for (int v = lane; v < nvec; v += 32) out[v] = make_uint4(0, 0, 0, 0);
      if (lane == 0) a.recv_meta[row] = make_int2(-1, -1);
      continue;
    }
    long long srow = row;
    if (a.per_token) {
      const int2 m = __ldcg(a.recv_meta + row);          // {source rank, source pair}
      srow = static_cast<long long>(m.x) * a.T + m.y / a.K;
      if (m.x < 0 || m.y < 0 || srow >= a.stage_rows) {   // never written: leave a zero row
        for (int v = lane; v < nvec; v += 32) out[v] = make_uint4(0, 0, 0, 0);
        continue;
      }
    }
    const uint2* __restrict__ q = reinterpret_cast<const uint2*>(a.recv_x + srow * a.H);
    const float* __restrict__ sc = a.recv_scale + srow * groups;
#pragma unroll 4
    for (int v = lane; v < nvec; v += 32) {
      const uint2 raw = __ldcg(q + v);
      const float s = __ldcg(sc + v / 16);
      const __nv_fp8x2_storage_t* p8 = reinterpret_cast<const __nv_fp8x2_storage_t*>(&raw);
      uint4 o;
      __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(p8[i], __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
        ob[i] = __floats2bfloat162_rn(f.x * s, f.y * s);
      }
      out[v] = o;
    }
  }
  if (a.ctas_done != nullptr) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (a.per_token) {       // every CTA polls every counter: only the last CTA of the grid may clear
        if (atomicAdd(a.ctas_done, 1u) == gridDim.x * gridDim.y - 1) {
          for (unsigned i = 0; i < gridDim.x; ++i) a.arrived[i] = 0u;
          a.ctas_done[0] = 0u;
        }
      } else if (atomicAdd(a.ctas_done + j, 1u) == gridDim.y - 1) {
        a.arrived[j] = 0u;
        a.ctas_done[j] = 0u;
      }
    }
  }
}

// out[r, i] = silu(in[r, i]) * in[r, I + i]; rows taken from n_rows_dev (device word).
__global__ void swiglu_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                              const int* n_rows_dev, int I) {
  const long long rows = *n_rows_dev;
  const long long vec_per_row = I / 8;
  const long long total = rows * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / vec_per_row, c = idx % vec_per_row;
    const uint4 g = *reinterpret_cast<const uint4*>(in + r * 2 * I + c * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(in + r * 2 * I + I + c * 8);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = __bfloat1622float2(gh[i]);
      const float2 b = __bfloat1622float2(uh[i]);
      oh[i] = __floats2bfloat162_rn(a.x / (1.f + __expf(-a.x)) * b.x,
                                    a.y / (1.f + __expf(-a.y)) * b.y);
    }
    *reinterpret_cast<uint4*>(out + r * I + c * 8) = o;
  }
}

// y[t, :] = sum_k w[t,k] * buf[t, k, :] (+ bias0[t, :] + bias1[t, :])   after every expert rank
// has reported in.  The two optional bias inputs [T, H] bf16 are those of the reference's
// reduction epilogue (datasets/example083_deepep_jit_combine_reduce_epilogue/nv/
// empty_deepep_jit_combine_reduce_epilogue.cu:28): a shared-expert output or a residual can be
// added here instead of in another pass over y.
// `done` = W words on this rank (one per expert rank); cleared by the last CTA.
__global__ void __launch_bounds__(256)
    moe_combine_reduce_kernel(const __nv_bfloat16* __restrict__ buf, const float* __restrict__ w,
                              const int* __restrict__ topk_idx, __nv_bfloat16* __restrict__ y,
                              int T, int K, int H, uint32_t* done, int world,
                              unsigned long long timeout_ns, uint32_t* status,
                              uint32_t* done_ctas, const __nv_bfloat16* __restrict__ bias0,
                              const __nv_bfloat16* __restrict__ bias1) {
  pdl_wait();                // chained with programmatic dependent launch: see prim/pdl.cuh
  pdl_launch_dependents();
  bool ok = true;
  if (threadIdx.x < static_cast<unsigned>(world))
    ok = wait_flag_ge_sys(done + threadIdx.x, 1u, timeout_ns, status, PH_MOE_COMBINE2,
                          threadIdx.x);
  if (__syncthreads_and(ok ? 1 : 0) != 0) {
    const int nvec = H / 8;
    const long long total = static_cast<long long>(T) * nvec;
    for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
         idx < total; idx += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long t = idx / nvec, v = idx % nvec;
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int b = 0; b < 2; ++b) {
        const __nv_bfloat16* bias = b == 0 ? bias0 : bias1;
        if (bias == nullptr) continue;
        const uint4 raw = *(reinterpret_cast<const uint4*>(bias + t * H) + v);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          acc[2 * i] += f.x;
          acc[2 * i + 1] += f.y;
        }
      }
      for (int k = 0; k < K; ++k) {
        if (topk_idx[t * K + k] < 0) continue;
        const float wk = w[t * K + k];
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(buf + (t * K + k) * H) + v);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          acc[2 * i] += wk * f.x;
          acc[2 * i + 1] += wk * f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      reinterpret_cast<uint4*>(y + t * H)[v] = o;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_ctas, 1u) == gridDim.x - 1) {
      for (int r = 0; r < world; ++r) done[r] = 0u;
      *done_ctas = 0u;
    }
  }
}

}  // namespace cb

using namespace cb;

extern "C" {

int cb_sizeof_moe_send_args() { return static_cast<int>(sizeof(MoeSendArgs)); }
int cb_sizeof_moe_recv_args() { return static_cast<int>(sizeof(MoeRecvArgs)); }

int cb_moe_dispatch_send(const MoeSendArgs* a, int slices, void* stream) {
  if (a->H % 256 != 0 || a->E % a->world != 0) {
    set_last_error("dispatch: hidden must be a multiple of 256 and experts divisible by ranks");
    return -1;
  }
  dim3 grid(a->E, slices < 1 ? 1 : slices);
  return launch_pdl(moe_dispatch_send_kernel, grid, dim3(256), 0,
                    static_cast<cudaStream_t>(stream), *a) == cudaSuccess
             ? 0
             : -1;
}

int cb_moe_recv_dequant(const MoeRecvArgs* a, int n_local_experts, int slices, void* stream) {
  if (a->per_token && (a->T < 1 || a->K < 1 || a->stage_rows < 1)) {
    set_last_error("receive: the per-token form needs T, K and stage_rows");
    return -1;
  }
  dim3 grid(n_local_experts, slices < 1 ? 1 : slices);
  return launch_pdl(moe_recv_dequant_kernel, grid, dim3(256), 0,
                    static_cast<cudaStream_t>(stream), *a) == cudaSuccess
             ? 0
             : -1;
}

int cb_moe_swiglu(const void* in, void* out, const void* n_rows_dev, int I, void* stream) {
  if (I % 8 != 0) return -1;
  swiglu_kernel<<<1184, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out),
      static_cast<const int*>(n_rows_dev), I);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// bias0 / bias1: optional [T, H] bf16 tensors added to the weighted sum (may be null).
int cb_moe_combine_reduce_bias(const void* buf, const void* w, const void* topk_idx, void* y,
                               int T, int K, int H, void* done, int world,
                               unsigned long long timeout_ns, void* status, void* done_ctas,
                               const void* bias0, const void* bias1, void* stream) {
  if (H % 8 != 0) return -1;
  return launch_pdl(moe_combine_reduce_kernel, dim3(592), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(buf),
                    static_cast<const float*>(w), static_cast<const int*>(topk_idx),
                    static_cast<__nv_bfloat16*>(y), T, K, H, static_cast<uint32_t*>(done), world,
                    timeout_ns, static_cast<uint32_t*>(status), static_cast<uint32_t*>(done_ctas),
                    static_cast<const __nv_bfloat16*>(bias0),
                    static_cast<const __nv_bfloat16*>(bias1)) == cudaSuccess
             ? 0
             : -1;
}

int cb_moe_combine_reduce(const void* buf, const void* w, const void* topk_idx, void* y, int T,
                          int K, int H, void* done, int world, unsigned long long timeout_ns,
                          void* status, void* done_ctas, void* stream) {
  return cb_moe_combine_reduce_bias(buf, w, topk_idx, y, T, K, H, done, world, timeout_ns, status,
                                    done_ctas, nullptr, nullptr, stream);
}

}  // extern "C"
