// Flash-attention forward, fifth design: the fourth design's pipeline (P kept in tensor memory as
// the A operand of the second MMA, K ring of 3 and V ring of 2 in shared memory) with the third
// design's softmax layout (two threads per query row, 16 softmax warps per CTA).
//
// Per tile the chain is S(j) -> softmax -> P(j) -> O += P V -> S(j+1); while one tile's warps run
// their softmax the tensor pipe works for the other tile, and with four softmax warps per
// scheduler the softmax of a block is short enough for the two chains to keep the pipe busy.
//
//   warp 0       TMA producer (Q tiles, K ring, V ring)
//   warp 1       MMA issuer
//   warps 2-9    softmax of tile 0, warps 10-17 of tile 1; the two warps with the same
//                (warp % 4) inside a tile share 32 rows and split the 128 keys of a block in
//                halves.  They agree on the reference maximum through a bf16 upper bound of
//                their half-row maxima in shared memory and a 64-thread named barrier; that
//                barrier also orders "both halves of S are in registers" before either partner
//                overwrites S columns with P.
//
// Same output contract as the other designs.  Every wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include <string>

#include "../gemm/tmap_host.h"
#include "../prim/tcgen05.cuh"
#include "../prim/tma.cuh"
#include "../symm/driver_api.h"

namespace cb {

static constexpr int F5_BM = 128;
static constexpr int F5_BN = 128;
static constexpr int F5_D = 128;
static constexpr int F5_SUB = 16384;
static constexpr int F5_TILE = 2 * F5_SUB;
static constexpr int F5_THREADS = 576;            // 2 + 16 warps
static constexpr float F5_RESCALE_THRESHOLD = 8.f;

struct Fa5Params {
  CUtensorMap tm_q, tm_k, tm_v;
  __nv_bfloat16* o;
  float* lse;
  int B, Sq, Skv, Hq, Hkv;
  int q_offset, kv_offset;
  int causal;
  float scale_log2;
  uint32_t* status;
};

static constexpr int F5_KST = 3, F5_VST = 2;

struct Fa5Ctl {
  uint64_t q_full;
  uint64_t k_full[F5_KST], k_empty[F5_KST];
  uint64_t v_full[F5_VST], v_empty[F5_VST];
  uint64_t s_full[2], p_full[2], pv_done[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Shared memory (all dynamic, so that its base is the 1024-byte aligned start of the CTA's
// window): Q 2 tiles | K 3 stages | V 2 stages | exchange 2 KB | control.
static constexpr int F5_XCHG_OFF = 7 * F5_TILE;
static constexpr int F5_XCHG_BYTES = 2048;        // [tile][parity][half][128 rows] bf16 / final fp32 sums
static constexpr int F5_CTL_OFF = F5_XCHG_OFF + F5_XCHG_BYTES;
static constexpr int F5_SMEM = F5_CTL_OFF + 160;
static_assert(sizeof(Fa5Ctl) <= 160, "control block");
static_assert(F5_SMEM <= 232448, "shared memory budget");

__device__ __forceinline__ uint64_t f5_mnmajor_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(F5_SUB >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__device__ __forceinline__ float f5_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint64_t f5_pack_u(uint32_t lo, uint32_t hi) {
  return static_cast<uint64_t>(lo) | (static_cast<uint64_t>(hi) << 32);
}
__device__ __forceinline__ uint64_t f5_pack(float lo, float hi) {
  return f5_pack_u(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ uint64_t f5_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f5_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float f5_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Barrier among the 64 threads (two warps) that share a set of rows.
__device__ __forceinline__ void f5_pair_sync(uint32_t id) {
  asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory");
}

__device__ __forceinline__ int f5_num_blocks(const Fa5Params& p, int tile128) {
  if (tile128 * F5_BM >= p.Sq) return 0;
  int nblk = (p.Skv + F5_BN - 1) / F5_BN;
  if (p.causal) {
    const int last_q = p.q_offset + (tile128 + 1) * F5_BM - 1;
    const int lim = last_q - p.kv_offset;
    if (lim < 0) return 0;
    const int c = lim / F5_BN + 1;
    if (c < nblk) nblk = c;
  }
  return nblk;
}

__global__ void __launch_bounds__(F5_THREADS, 1) fa_fwd5_kernel(const __grid_constant__ Fa5Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + 2 * F5_TILE;
  uint8_t* sV = sK + F5_KST * F5_TILE;
  Fa5Ctl& ctl = *reinterpret_cast<Fa5Ctl*>(smem + F5_CTL_OFF);
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const int q_pair = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int nblk0 = f5_num_blocks(p, 2 * q_pair), nblk1 = f5_num_blocks(p, 2 * q_pair + 1);
  const int nblk_max = nblk0 > nblk1 ? nblk0 : nblk1;
  // The swizzled tiles need a 1024-byte aligned base; refuse to run otherwise.
  const bool aligned = (smem_u32(smem) & 1023u) == 0u;

  if (threadIdx.x == 0) {
    mbar_init(&ctl.q_full, 1);
    for (int i = 0; i < F5_KST; ++i) {
      mbar_init(&ctl.k_full[i], 1);
      mbar_init(&ctl.k_empty[i], 1);
    }
    for (int i = 0; i < F5_VST; ++i) {
      mbar_init(&ctl.v_full[i], 1);
      mbar_init(&ctl.v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl.s_full[i], 1);
      mbar_init(&ctl.p_full[i], 8);
      mbar_init(&ctl.pv_done[i], 1);
    }
    ctl.abort_flag = 0;
    if (!aligned) {
      ctl.abort_flag = 1;
      report_status(p.status, CB_BAD_ARGUMENT, 0, 0xE00);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&ctl.tmem_base);
  const bool run = aligned && nblk_max > 0;

  if (warp == 0) {
    if (lane == 0 && run) {
      // ---------------------------------------------------------------- producer
      mbar_arrive_expect_tx(&ctl.q_full, 2 * F5_TILE);
      const int qrow = batch * p.Sq + q_pair * 2 * F5_BM;
      for (int t = 0; t < 2; ++t) {
        tma_load_3d(sQ + t * F5_TILE, &p.tm_q, 0, head, qrow + t * F5_BM, &ctl.q_full);
        tma_load_3d(sQ + t * F5_TILE + F5_SUB, &p.tm_q, 64, head, qrow + t * F5_BM, &ctl.q_full);
      }
      int jk = 0, jv = 0;
      uint32_t idle = 0;
      uint64_t t0 = 0;
      while (jk < nblk_max || jv < nblk_max) {
        bool progress = false;
        if (jk < nblk_max) {
          const int s = jk % F5_KST, use = jk / F5_KST;
          if (use == 0 || mbar_try_wait(&ctl.k_empty[s], (use - 1) & 1)) {
            const int krow = batch * p.Skv + jk * F5_BN;
            mbar_arrive_expect_tx(&ctl.k_full[s], F5_TILE);
            tma_load_3d(sK + s * F5_TILE, &p.tm_k, 0, kv_head, krow, &ctl.k_full[s]);
            tma_load_3d(sK + s * F5_TILE + F5_SUB, &p.tm_k, 64, kv_head, krow, &ctl.k_full[s]);
            ++jk;
            progress = true;
          }
        }
        if (jv < nblk_max && jv < jk) {
          const int s = jv % F5_VST, use = jv / F5_VST;
          if (use == 0 || mbar_try_wait(&ctl.v_empty[s], (use - 1) & 1)) {
            const int vrow = batch * p.Skv + jv * F5_BN;
            mbar_arrive_expect_tx(&ctl.v_full[s], F5_TILE);
            tma_load_3d(sV + s * F5_TILE, &p.tm_v, 0, kv_head, vrow, &ctl.v_full[s]);
            tma_load_3d(sV + s * F5_TILE + F5_SUB, &p.tm_v, 64, kv_head, vrow, &ctl.v_full[s]);
            ++jv;
            progress = true;
          }
        }
        if (progress) {
          idle = 0;
          continue;
        }
        if ((++idle & 255u) == 0u) {
          if (*reinterpret_cast<volatile int*>(&ctl.abort_flag) != 0) break;
          const uint64_t now = globaltimer_ns();
          if (t0 == 0 || idle == 256u) t0 = now;
          if (now - t0 > CB_MBAR_TIMEOUT_NS) {
            ctl.abort_flag = 1;
            report_status(p.status, CB_TIMEOUT_MBARRIER, 0, 0xE01);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && run) {
      // --------------------------------------------------------------------- MMA
      constexpr uint32_t idesc_s = make_idesc(128, 128, 1u);
      constexpr uint32_t idesc_pv = make_idesc(128, 128, 1u) | (1u << 16);  // B (= V) is MN-major
      const int nb[2] = {nblk0, nblk1};
      bool ok = mbar_wait(&ctl.q_full, 0, &ctl.abort_flag, p.status, 0xE10);
      auto issue_qk = [&](int t, int j) -> bool {
        const int s = j % F5_KST;
        if (!mbar_wait(&ctl.k_full[s], (j / F5_KST) & 1, &ctl.abort_flag, p.status, 0xE11)) return false;
        tc_fence_after_sync();
        const uint32_t qa = smem_u32(sQ + t * F5_TILE), ka = smem_u32(sK + s * F5_TILE);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a_desc = make_sw128_kmajor_desc(qa + (kk >> 2) * F5_SUB) + 2u * (kk & 3);
          const uint64_t b_desc = make_sw128_kmajor_desc(ka + (kk >> 2) * F5_SUB) + 2u * (kk & 3);
          mma_bf16_ss(tmem + 256u * t, a_desc, b_desc, idesc_s, kk > 0 ? 1u : 0u);
        }
        mma_commit(&ctl.s_full[t]);
        return true;
      };
      auto issue_pv = [&](int t, int j) -> bool {
        const int s = j % F5_VST;
        if (!mbar_wait(&ctl.p_full[t], j & 1, &ctl.abort_flag, p.status, 0xE20 + t)) return false;
        if (!mbar_wait(&ctl.v_full[s], (j / F5_VST) & 1, &ctl.abort_flag, p.status, 0xE22)) return false;
        tc_fence_after_sync();
        const uint32_t va = smem_u32(sV + s * F5_TILE);
        const uint32_t d = tmem + 256u * t + 128u;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A = P_t from tensor memory: 16 keys = 8 columns of bf16 pairs per step.
          const uint64_t b_desc = f5_mnmajor_desc(va + kk * 2048);
          mma_bf16_ts(d, tmem + 256u * t + 8u * kk, b_desc, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        }
        mma_commit(&ctl.pv_done[t]);
        return true;
      };
      // prologue: S_t(0) of both tiles
      for (int t = 0; ok && t < 2; ++t)
        if (nb[t] > 0) ok = issue_qk(t, 0);
      if (ok) mma_commit(&ctl.k_empty[0]);
      for (int j = 0; ok && j < nblk_max; ++j) {
        for (int t = 0; ok && t < 2; ++t) {
          if (j >= nb[t]) continue;
          ok = issue_pv(t, j);
          if (ok && j + 1 < nb[t]) ok = issue_qk(t, j + 1);
        }
        if (!ok) break;
        mma_commit(&ctl.v_empty[j % F5_VST]);
        if (j + 1 < nblk_max) mma_commit(&ctl.k_empty[(j + 1) % F5_KST]);
      }
    }
  } else if (aligned) {
    // ------------------------------------------------------------------- softmax
    const uint32_t w = warp - 2u;              // 0..15
    const int t = static_cast<int>(w >> 3);    // query tile
    const uint32_t h = (w >> 2) & 1u;          // which 64 keys of every block
    const uint32_t q = warp & 3u;              // TMEM lane quadrant this warp may touch
    const int nblk = t ? nblk1 : nblk0;
    const uint32_t r = q * 32u + lane;         // row inside the tile
    const uint32_t lane_addr = (q * 32u) << 16;
    const uint32_t tS = tmem + 256u * t + lane_addr + 64u * h;
    const uint32_t tO = tmem + 256u * t + 128u + lane_addr + 64u * h;
    const int tile128 = 2 * q_pair + t;
    const int q_pos = p.q_offset + tile128 * F5_BM + static_cast<int>(r);
    const uint32_t tP = tmem + 256u * t + lane_addr + 32u * h;   // P: first 64 columns of S
    const uint32_t pair_bar = 1u + static_cast<uint32_t>(t) * 4u + q;
    __nv_bfloat16* xchg = reinterpret_cast<__nv_bfloat16*>(smem + F5_XCHG_OFF);
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      if (ok && !mbar_wait(&ctl.s_full[t], j & 1, &ctl.abort_flag, p.status, 0xE30 + t)) ok = false;
      uint32_t s[64];
      if (ok) {
        tc_fence_after_sync();
        tmem_ld_32x32_at(tS, &s[0]);
        tmem_ld_32x32_at(tS + 32u, &s[32]);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) s[i] = 0xff800000u;
      }
      const int key0 = p.kv_offset + j * F5_BN + 64 * static_cast<int>(h);
      const int kv_left = p.Skv - j * F5_BN - 64 * static_cast<int>(h);
      const bool need_mask = kv_left < 64 ||
                             (p.causal && key0 + 63 > p.q_offset + tile128 * F5_BM);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (!(i < kv_left && (!p.causal || key0 + i <= q_pos))) s[i] = 0xff800000u;
      }
      float mx8[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx8[i] = fmaxf(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1]));
#pragma unroll
      for (int i = 16; i < 64; i += 2)
        mx8[(i >> 1) & 7] = f5_max3(mx8[(i >> 1) & 7], __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
      const float mx_half = f5_max3(fmaxf(f5_max3(mx8[0], mx8[1], mx8[2]), f5_max3(mx8[3], mx8[4], mx8[5])),
                                    mx8[6], mx8[7]) * p.scale_log2;
      // Publish an upper bound of this half's maximum; both partners read both values.
      // (Every thread reaches this barrier in every block, also after a failed wait.)
      __nv_bfloat16* slot = xchg + ((t * 2 + (j & 1)) * 2) * 128;
      slot[h * 128 + r] = __float2bfloat16_ru(mx_half);
      f5_pair_sync(pair_bar);
      const float mx_s = fmaxf(__bfloat162float(slot[r]), __bfloat162float(slot[128 + r]));
      if (!ok) continue;
      const bool grow = mx_s > m_ref + F5_RESCALE_THRESHOLD || (m_ref == -INFINITY && mx_s > -INFINITY);
      const bool any_grow = __any_sync(0xffffffffu, grow);
      float alpha = 1.f;
      if (any_grow) {
        const float m_new = fmaxf(m_ref, mx_s);
        alpha = m_ref == -INFINITY ? 0.f : f5_ex2(m_ref - m_new);
        m_ref = m_new;
        l *= alpha;
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      const uint64_t scale2 = f5_pack(p.scale_log2, p.scale_log2), negm2 = f5_pack(-m_use, -m_use);
      uint64_t sum4[4] = {0ull, 0ull, 0ull, 0ull};
      uint32_t packed[32];
#pragma unroll
      for (int i = 0; i < 64; i += 2) {
        const uint64_t y = f5_fma2(f5_pack_u(s[i], s[i + 1]), scale2, negm2);
        const float p0 = f5_ex2(__uint_as_float(static_cast<uint32_t>(y)));
        const float p1 = f5_ex2(__uint_as_float(static_cast<uint32_t>(y >> 32)));
        sum4[(i >> 1) & 3] = f5_add2(sum4[(i >> 1) & 3], f5_pack(p0, p1));
        __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&hh);
      }
      {
        const uint64_t a = f5_add2(f5_add2(sum4[0], sum4[1]), f5_add2(sum4[2], sum4[3]));
        l += __uint_as_float(static_cast<uint32_t>(a)) + __uint_as_float(static_cast<uint32_t>(a >> 32));
      }
      // S(j) complete implies P(j-1) V(j-1) complete (one issuing thread, commits cover all
      // earlier MMAs): O is stable and the P columns may be overwritten.  The pair barrier
      // above ordered the partner's S loads before this store.
      if (any_grow && j > 0) {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tO + c * 32u, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(tO + c * 32u, o);
        }
      }
      // P(j): row r = lane r; this half's 64 keys are 32 columns of bf16 pairs.
      tmem_st_32x32(tP, packed);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.p_full[t]);
    }
    // ------------------------------------------------------------------ epilogue
    const int row = tile128 * F5_BM + static_cast<int>(r);
    if (ok && nblk > 0)
      ok = mbar_wait(&ctl.pv_done[t], (nblk - 1) & 1, &ctl.abort_flag, p.status, 0xE34 + t);
    // Row sum = sum of the two halves: one fp32 exchange through the same 2 KB.
    float* lsum = reinterpret_cast<float*>(smem + F5_XCHG_OFF);
    f5_pair_sync(pair_bar);                       // nobody still reads the bf16 maxima
    lsum[(t * 2 + h) * 128 + r] = l;
    f5_pair_sync(pair_bar);
    const float l_row = lsum[(t * 2) * 128 + r] + lsum[(t * 2 + 1) * 128 + r];
    if (ok && tile128 * F5_BM < p.Sq) {
      tc_fence_after_sync();
      const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
      __nv_bfloat16* dst = p.o + ((static_cast<size_t>(batch) * p.Sq + row) * p.Hq + head) * F5_D + 64 * h;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t o[32];
        if (nblk > 0) {
          tmem_ld_32x32(tO + c * 32u, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (row < p.Sq) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              hh[k] = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * k]) * inv,
                                            __uint_as_float(o[i + 2 * k + 1]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
          }
        }
      }
      if (row < p.Sq && h == 0)
        p.lse[(static_cast<size_t>(batch) * p.Hq + head) * p.Sq + row] =
            l_row > 0.f ? (m_ref * 0.6931471805599453f + logf(l_row)) : -INFINITY;
    }
  }
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (*reinterpret_cast<volatile int*>(&ctl.abort_flag) != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace cb

using namespace cb;

int cb_attn_make_tmap_bshd(CUtensorMap* out, const void* base, int rows, int heads);

extern "C" {

// Same contract as cb_attn_fwd (fa_fwd.cu).
int cb_attn_fwd5(const void* q, const void* k, const void* v, void* o, void* lse, int B, int Sq,
                 int Skv, int Hq, int Hkv, int q_offset, int kv_offset, int causal, float scale,
                 void* status, void* stream) {
  if (B < 1 || Sq < 1 || Skv < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0) {
    set_last_error("attention: bad shape (Hq must be a multiple of Hkv)");
    return -1;
  }
  Fa5Params p;
  if (cb_attn_make_tmap_bshd(&p.tm_q, q, B * Sq, Hq)) return -1;
  if (cb_attn_make_tmap_bshd(&p.tm_k, k, B * Skv, Hkv)) return -1;
  if (cb_attn_make_tmap_bshd(&p.tm_v, v, B * Skv, Hkv)) return -1;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = static_cast<float*>(lse);
  p.B = B;
  p.Sq = Sq;
  p.Skv = Skv;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.q_offset = q_offset;
  p.kv_offset = kv_offset;
  p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = static_cast<uint32_t*>(status);
  cudaError_t e = cudaFuncSetAttribute(fa_fwd5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       F5_SMEM);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    return -1;
  }
  dim3 grid((Sq + 2 * F5_BM - 1) / (2 * F5_BM), Hq, B);
  fa_fwd5_kernel<<<grid, F5_THREADS, F5_SMEM, static_cast<cudaStream_t>(stream)>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(std::string("attention launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // extern "C"
