// Fused tensor-parallel QK-RMSNorm: the heads of Q and K are sharded over the
// ranks, RMSNorm needs the sum of squares over ALL heads of a token, and the
// whole thing is ONE kernel: local partial sums, a push all-reduce of two floats
// per token through peer memory, scale, in-place multiply by the norm weight.
//
// Same algorithm as the reference's fused kernel (stages at
// datasets/example102_sglang_qknorm_fused_hard/empty_sglang_qknorm_fused_hard.cu:9-41; kernel
// shape at datasets/example101_sglang_qknorm_fused_easy/empty_sglang_qknorm_fused_easy.cu:132-209):
// one CTA per token, an 8-byte push per peer, zero as the "not written yet"
// sentinel, epoch-rotated slots.  Differences: the world size is a run-time value,
// the epoch lives in device memory (bumped by the last CTA, so replaying the launch
// needs no host state), and the poll is bounded and reports a status word.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../prim/barrier.cuh"

namespace cb {
void set_last_error(const std::string& s);

enum : uint32_t { PH_QKNORM = 56 };

struct QkNormArgs {
  __nv_bfloat16* q;          // [tokens, q_local] in place
  __nv_bfloat16* k;          // [tokens, k_local] in place
  const __nv_bfloat16* wq;   // [q_local] this rank's slice of the norm weight
  const __nv_bfloat16* wk;   // [k_local]
  float2* buf[CB_MAX_RANKS]; // per rank: [2 epochs][max_tokens][world] float2
  uint32_t* seq;             // {call counter, CTAs done} local device words
  int rank, world, tokens, max_tokens, q_local, k_local;
  float eps;
  unsigned long long timeout_ns;
  uint32_t* status;
};

__global__ void __launch_bounds__(256) qknorm_kernel(const __grid_constant__ QkNormArgs a,
                                                     const QkNormArgs* emu) {
  const QkNormArgs& p = emu != nullptr ? emu[blockIdx.y] : a;
  const int token = blockIdx.x;
  const uint32_t epoch = ld_volatile(p.seq) & 1u;
  const int qv = p.q_local / 8, kv = p.k_local / 8;
  uint4* qrow = reinterpret_cast<uint4*>(p.q + static_cast<size_t>(token) * p.q_local);
  uint4* krow = reinterpret_cast<uint4*>(p.k + static_cast<size_t>(token) * p.k_local);
  // Stage 1: local sums of squares
  float sq = 0.f, sk = 0.f;
  for (int v = threadIdx.x; v < qv + kv; v += blockDim.x) {
    const uint4 raw = v < qv ? qrow[v] : krow[v - qv];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      s += f.x * f.x + f.y * f.y;
    }
    if (v < qv) sq += s; else sk += s;
  }
  __shared__ float red[2][8];
  __shared__ float scale[2];
  __shared__ int failed;
  for (int o = 16; o > 0; o >>= 1) {
    sq += __shfl_xor_sync(0xffffffffu, sq, o);
    sk += __shfl_xor_sync(0xffffffffu, sk, o);
  }
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = sq;
    red[1][threadIdx.x >> 5] = sk;
  }
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  // Stage 2: push my partial sums to every rank, poll until everyone's arrived
  if (threadIdx.x < 32) {
    float tq = 0.f, tk = 0.f;
    for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) {
      tq += red[0][w];
      tk += red[1][w];
    }
    const int lane = threadIdx.x;
    float gq = 0.f, gk = 0.f;
    if (lane < p.world) {
      const size_t slot = (static_cast<size_t>(epoch) * p.max_tokens + token) * p.world;
      // +tiny: a written slot is never zero, so zero can mean "not yet"
      st_volatile_v2f(p.buf[lane] + slot + p.rank, make_float2(tq + 1e-30f, tk + 1e-30f));
      float2* mine = p.buf[p.rank] + slot + lane;
      float2 got = ld_volatile_v2f(mine);
      if (got.x == 0.f || got.y == 0.f) {
        const uint64_t t0 = globaltimer_ns();
        for (uint32_t it = 0;; ++it) {
          got = ld_volatile_v2f(mine);
          if (got.x != 0.f && got.y != 0.f) break;
          if ((it & 63u) == 63u && globaltimer_ns() - t0 > p.timeout_ns) {
            report_status(p.status, CB_TIMEOUT_PEER_FLAG, PH_QKNORM, lane);
            failed = 1;
            break;
          }
        }
      }
      gq = got.x;
      gk = got.y;
      st_volatile_v2f(mine, make_float2(0.f, 0.f));  // clean for the call after next
    }
    for (int o = 16; o > 0; o >>= 1) {
      gq += __shfl_xor_sync(0xffffffffu, gq, o);
      gk += __shfl_xor_sync(0xffffffffu, gk, o);
    }
    if (lane == 0) {
      // Stage 3
      scale[0] = rsqrtf(gq / (static_cast<float>(p.q_local) * p.world) + p.eps);
      scale[1] = rsqrtf(gk / (static_cast<float>(p.k_local) * p.world) + p.eps);
    }
  }
  __syncthreads();
  // Stage 4: in-place scale * weight
  if (!failed) {
    const uint4* wq = reinterpret_cast<const uint4*>(p.wq);
    const uint4* wk = reinterpret_cast<const uint4*>(p.wk);
    for (int v = threadIdx.x; v < qv + kv; v += blockDim.x) {
      const bool isq = v < qv;
      uint4* ptr = isq ? qrow + v : krow + (v - qv);
      const uint4 raw = *ptr;
      const uint4 wr = isq ? wq[v] : wk[v - qv];
      const float s = scale[isq ? 0 : 1];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wr);
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        const float2 g = __bfloat1622float2(wh[i]);
        oh[i] = __floats2bfloat162_rn(f.x * s * g.x, f.y * s * g.y);
      }
      *ptr = o;
    }
  }
  // last CTA of this (virtual) rank bumps the epoch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.seq + 1, 1u) == gridDim.x - 1) {
      p.seq[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.seq) = ld_volatile(p.seq) + 1u;
    }
  }
}

}  // namespace cb

using namespace cb;

extern "C" {

int cb_sizeof_qknorm_args() { return static_cast<int>(sizeof(QkNormArgs)); }

// n == 1: a real rank.  n > 1: n virtual ranks in one cooperative launch (`emu_table` =
// device copy of the n argument blocks).
int cb_qknorm(const QkNormArgs* args, int n, const void* emu_table, void* stream) {
  const QkNormArgs& a = args[0];
  if (a.q_local % 8 != 0 || a.k_local % 8 != 0 || a.tokens < 1 || a.tokens > a.max_tokens) {
    set_last_error("qknorm: head slices must be multiples of 8 and tokens <= max_tokens");
    return -1;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (n > 1) {
    const QkNormArgs* emu = static_cast<const QkNormArgs*>(emu_table);
    void* params[] = {const_cast<QkNormArgs*>(&a), &emu};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(qknorm_kernel), dim3(a.tokens, n),
                                    dim3(256), params, 0, st);
  } else {
    qknorm_kernel<<<a.tokens, 256, 0, st>>>(a, nullptr);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    set_last_error(std::string("qknorm launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // extern "C"
