// Flash-attention forward, third design: as the second (two query tiles of 128 rows per CTA,
// O accumulated in tensor memory, scores read once) but with TWO threads per query row, each
// owning 64 of the 128 keys of a block: 16 softmax warps per CTA instead of 8.  The second
// design is bound by issue slots and latency of its softmax warps (two per scheduler); four
// per scheduler hide the TMEM-load, SFU and barrier latencies of one another.
//
//   warp 0       TMA producer (Q tiles, K two stages, V one stage)
//   warp 1       MMA issuer (S_t = Q_t K^T, O_t += P_t V)
//   warps 2-9    softmax of tile 0, warps 10-17 of tile 1.  Warp w may touch TMEM lanes
//                32 (w % 4) ... + 31, so the two warps with the same (w % 4) inside a tile
//                share the rows and split the columns: half h = keys 64 h ... 64 h + 63.
//
// The two threads of a row must use the same reference maximum (their P values feed the same
// accumulation), so every block they exchange their half-row maxima through shared memory and
// a 64-thread named barrier; both read BOTH published values, so they decide identically.
// The values travel as bf16 rounded up (an upper bound of the maximum is all the lazy-rescale
// rule needs); the two halves of the row sum are added once at the end.
//
// Same output contract as the other designs (normalised O of this key/value chunk + row-wise
// log-sum-exp).  Every wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include <string>

#include "../gemm/tmap_host.h"
#include "../prim/tcgen05.cuh"
#include "../prim/tma.cuh"
#include "../symm/driver_api.h"

namespace cb {

static constexpr int F3_BM = 128;
static constexpr int F3_BN = 128;
static constexpr int F3_D = 128;
static constexpr int F3_SUB = 16384;
static constexpr int F3_TILE = 2 * F3_SUB;
static constexpr int F3_THREADS = 576;            // 2 + 16 warps
static constexpr float F3_RESCALE_THRESHOLD = 8.f;

struct Fa3Params {
  CUtensorMap tm_q, tm_k, tm_v;
  __nv_bfloat16* o;
  float* lse;
  int B, Sq, Skv, Hq, Hkv;
  int q_offset, kv_offset;
  int causal;
  float scale_log2;
  uint32_t* status;
};

struct Fa3Ctl {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2];
  uint64_t v_full, v_empty;
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full[2], pv_done[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Shared memory (all dynamic, so that its base is the 1024-byte aligned start of the CTA's
// window): Q 2 tiles | K 2 stages | V 1 stage | P 2 tiles | exchange 2 KB | control.
static constexpr int F3_XCHG_OFF = 7 * F3_TILE;
static constexpr int F3_XCHG_BYTES = 2048;        // [tile][parity][half][128 rows] bf16 / final fp32 sums
static constexpr int F3_CTL_OFF = F3_XCHG_OFF + F3_XCHG_BYTES;
static constexpr int F3_SMEM = F3_CTL_OFF + 128;
static_assert(sizeof(Fa3Ctl) <= 128, "control block");
static_assert(F3_SMEM <= 232448, "shared memory budget");

__device__ __forceinline__ uint64_t f3_mnmajor_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(F3_SUB >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__device__ __forceinline__ float f3_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint64_t f3_pack_u(uint32_t lo, uint32_t hi) {
  return static_cast<uint64_t>(lo) | (static_cast<uint64_t>(hi) << 32);
}
__device__ __forceinline__ uint64_t f3_pack(float lo, float hi) {
  return f3_pack_u(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ uint64_t f3_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f3_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float f3_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Barrier among the 64 threads (two warps) that share a set of rows.
__device__ __forceinline__ void f3_pair_sync(uint32_t id) {
  asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory");
}

__device__ __forceinline__ int f3_num_blocks(const Fa3Params& p, int tile128) {
  if (tile128 * F3_BM >= p.Sq) return 0;
  int nblk = (p.Skv + F3_BN - 1) / F3_BN;
  if (p.causal) {
    const int last_q = p.q_offset + (tile128 + 1) * F3_BM - 1;
    const int lim = last_q - p.kv_offset;
    if (lim < 0) return 0;
    const int c = lim / F3_BN + 1;
    if (c < nblk) nblk = c;
  }
  return nblk;
}

__global__ void __launch_bounds__(F3_THREADS, 1) fa_fwd3_kernel(const __grid_constant__ Fa3Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + 2 * F3_TILE;
  uint8_t* sV = sK + 2 * F3_TILE;
  uint8_t* sP = sV + F3_TILE;
  Fa3Ctl& ctl = *reinterpret_cast<Fa3Ctl*>(smem + F3_CTL_OFF);
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const int q_pair = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int nblk0 = f3_num_blocks(p, 2 * q_pair), nblk1 = f3_num_blocks(p, 2 * q_pair + 1);
  const int nblk_max = nblk0 > nblk1 ? nblk0 : nblk1;
  // The swizzled tiles need a 1024-byte aligned base; refuse to run otherwise.
  const bool aligned = (smem_u32(smem) & 1023u) == 0u;

  if (threadIdx.x == 0) {
    mbar_init(&ctl.q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl.k_full[i], 1);
      mbar_init(&ctl.k_empty[i], 1);
      mbar_init(&ctl.s_full[i], 1);
      mbar_init(&ctl.s_empty[i], 8);
      mbar_init(&ctl.p_full[i], 8);
      mbar_init(&ctl.pv_done[i], 1);
    }
    mbar_init(&ctl.v_full, 1);
    mbar_init(&ctl.v_empty, 1);
    ctl.abort_flag = 0;
    if (!aligned) {
      ctl.abort_flag = 1;
      report_status(p.status, CB_BAD_ARGUMENT, 0, 0xC00);
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
      mbar_arrive_expect_tx(&ctl.q_full, 2 * F3_TILE);
      const int qrow = batch * p.Sq + q_pair * 2 * F3_BM;
      for (int t = 0; t < 2; ++t) {
        tma_load_3d(sQ + t * F3_TILE, &p.tm_q, 0, head, qrow + t * F3_BM, &ctl.q_full);
        tma_load_3d(sQ + t * F3_TILE + F3_SUB, &p.tm_q, 64, head, qrow + t * F3_BM, &ctl.q_full);
      }
      int jk = 0, jv = 0;
      uint32_t idle = 0;
      uint64_t t0 = 0;
      while (jk < nblk_max || jv < nblk_max) {
        bool progress = false;
        if (jk < nblk_max) {
          const int s = jk & 1;
          if (jk < 2 || mbar_try_wait(&ctl.k_empty[s], ((jk >> 1) - 1) & 1)) {
            const int krow = batch * p.Skv + jk * F3_BN;
            mbar_arrive_expect_tx(&ctl.k_full[s], F3_TILE);
            tma_load_3d(sK + s * F3_TILE, &p.tm_k, 0, kv_head, krow, &ctl.k_full[s]);
            tma_load_3d(sK + s * F3_TILE + F3_SUB, &p.tm_k, 64, kv_head, krow, &ctl.k_full[s]);
            ++jk;
            progress = true;
          }
        }
        if (jv < nblk_max && jv < jk) {
          if (jv < 1 || mbar_try_wait(&ctl.v_empty, (jv - 1) & 1)) {
            const int vrow = batch * p.Skv + jv * F3_BN;
            mbar_arrive_expect_tx(&ctl.v_full, F3_TILE);
            tma_load_3d(sV, &p.tm_v, 0, kv_head, vrow, &ctl.v_full);
            tma_load_3d(sV + F3_SUB, &p.tm_v, 64, kv_head, vrow, &ctl.v_full);
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
            report_status(p.status, CB_TIMEOUT_MBARRIER, 0, 0xC01);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && run) {
      // --------------------------------------------------------------------- MMA
      constexpr uint32_t idesc_s = make_idesc(128, 128, 1u);
      constexpr uint32_t idesc_pv = make_idesc(128, 128, 1u) | (1u << 16);
      const int nb[2] = {nblk0, nblk1};
      bool ok = mbar_wait(&ctl.q_full, 0, &ctl.abort_flag, p.status, 0xC10);
      auto issue_pv = [&](int t, int j) -> bool {
        if (!mbar_wait(&ctl.p_full[t], j & 1, &ctl.abort_flag, p.status, 0xC20 + t)) return false;
        if (!mbar_wait(&ctl.v_full, j & 1, &ctl.abort_flag, p.status, 0xC22)) return false;
        tc_fence_after_sync();
        const uint32_t pa = smem_u32(sP + t * F3_TILE), va = smem_u32(sV);
        const uint32_t d = tmem + 256u * t + 128u;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a_desc = make_sw128_kmajor_desc(pa + (kk >> 2) * F3_SUB) + 2u * (kk & 3);
          const uint64_t b_desc = f3_mnmajor_desc(va + kk * 2048);
          mma_bf16_ss(d, a_desc, b_desc, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        }
        mma_commit(&ctl.pv_done[t]);
        return true;
      };
      for (int j = 0; ok && j < nblk_max; ++j) {
        const int s = j & 1;
        ok = mbar_wait(&ctl.k_full[s], (j >> 1) & 1, &ctl.abort_flag, p.status, 0xC11);
        for (int t = 0; ok && t < 2; ++t) {
          if (j >= nb[t]) continue;
          ok = mbar_wait(&ctl.s_empty[t], (j & 1) ^ 1u, &ctl.abort_flag, p.status, 0xC12 + t);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t qa = smem_u32(sQ + t * F3_TILE), ka = smem_u32(sK + s * F3_TILE);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t a_desc = make_sw128_kmajor_desc(qa + (kk >> 2) * F3_SUB) + 2u * (kk & 3);
            const uint64_t b_desc = make_sw128_kmajor_desc(ka + (kk >> 2) * F3_SUB) + 2u * (kk & 3);
            mma_bf16_ss(tmem + 256u * t, a_desc, b_desc, idesc_s, kk > 0 ? 1u : 0u);
          }
          mma_commit(&ctl.s_full[t]);
        }
        if (!ok) break;
        mma_commit(&ctl.k_empty[s]);
        if (j > 0) {
          for (int t = 0; ok && t < 2; ++t)
            if (j - 1 < nb[t]) ok = issue_pv(t, j - 1);
          if (ok) mma_commit(&ctl.v_empty);
        }
      }
      for (int t = 0; ok && t < 2; ++t)
        if (nblk_max - 1 < nb[t]) ok = issue_pv(t, nblk_max - 1);
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
    const int q_pos = p.q_offset + tile128 * F3_BM + static_cast<int>(r);
    uint8_t* sPt = sP + t * F3_TILE + h * F3_SUB;          // this half = one 64-key sub-tile
    const uint32_t pair_bar = 1u + static_cast<uint32_t>(t) * 4u + q;
    __nv_bfloat16* xchg = reinterpret_cast<__nv_bfloat16*>(smem + F3_XCHG_OFF);
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      if (ok && !mbar_wait(&ctl.s_full[t], j & 1, &ctl.abort_flag, p.status, 0xC30 + t)) ok = false;
      uint32_t s[64];
      if (ok) {
        tc_fence_after_sync();
        tmem_ld_32x32_at(tS, &s[0]);
        tmem_ld_32x32_at(tS + 32u, &s[32]);
        tmem_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.s_empty[t]);
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) s[i] = 0xff800000u;
      }
      const int key0 = p.kv_offset + j * F3_BN + 64 * static_cast<int>(h);
      const int kv_left = p.Skv - j * F3_BN - 64 * static_cast<int>(h);
      const bool need_mask = kv_left < 64 ||
                             (p.causal && key0 + 63 > p.q_offset + tile128 * F3_BM);
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
        mx8[(i >> 1) & 7] = f3_max3(mx8[(i >> 1) & 7], __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
      const float mx_half = f3_max3(fmaxf(f3_max3(mx8[0], mx8[1], mx8[2]), f3_max3(mx8[3], mx8[4], mx8[5])),
                                    mx8[6], mx8[7]) * p.scale_log2;
      // Publish an upper bound of this half's maximum; both partners read both values.
      // (Every thread reaches this barrier in every block, also after a failed wait.)
      __nv_bfloat16* slot = xchg + ((t * 2 + (j & 1)) * 2) * 128;
      slot[h * 128 + r] = __float2bfloat16_ru(mx_half);
      f3_pair_sync(pair_bar);
      const float mx_s = fmaxf(__bfloat162float(slot[r]), __bfloat162float(slot[128 + r]));
      if (!ok) continue;
      const bool grow = mx_s > m_ref + F3_RESCALE_THRESHOLD || (m_ref == -INFINITY && mx_s > -INFINITY);
      const bool any_grow = __any_sync(0xffffffffu, grow);
      float alpha = 1.f;
      if (any_grow) {
        const float m_new = fmaxf(m_ref, mx_s);
        alpha = m_ref == -INFINITY ? 0.f : f3_ex2(m_ref - m_new);
        m_ref = m_new;
        l *= alpha;
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      const uint64_t scale2 = f3_pack(p.scale_log2, p.scale_log2), negm2 = f3_pack(-m_use, -m_use);
      uint64_t sum4[4] = {0ull, 0ull, 0ull, 0ull};
      uint32_t packed[32];
#pragma unroll
      for (int i = 0; i < 64; i += 2) {
        const uint64_t y = f3_fma2(f3_pack_u(s[i], s[i + 1]), scale2, negm2);
        const float p0 = f3_ex2(__uint_as_float(static_cast<uint32_t>(y)));
        const float p1 = f3_ex2(__uint_as_float(static_cast<uint32_t>(y >> 32)));
        sum4[(i >> 1) & 3] = f3_add2(sum4[(i >> 1) & 3], f3_pack(p0, p1));
        __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&hh);
      }
      {
        const uint64_t a = f3_add2(f3_add2(sum4[0], sum4[1]), f3_add2(sum4[2], sum4[3]));
        l += __uint_as_float(static_cast<uint32_t>(a)) + __uint_as_float(static_cast<uint32_t>(a >> 32));
      }
      // P(j-1) V(j-1) must have completed: it read the P buffer and wrote O.
      if (!mbar_wait(&ctl.pv_done[t], (j & 1) ^ 1u, &ctl.abort_flag, p.status, 0xC32 + t)) {
        ok = false;
        continue;
      }
      if (any_grow && j > 0) {
        tc_fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tO + c * 32u, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(tO + c * 32u, o);
        }
        tmem_wait_st();
      }
#pragma unroll
      for (int ci = 0; ci < 8; ++ci) {
        uint8_t* dst = sPt + r * 128u + ((static_cast<uint32_t>(ci) ^ (r & 7u)) * 16u);
        *reinterpret_cast<uint4*>(dst) = make_uint4(packed[ci * 4], packed[ci * 4 + 1],
                                                    packed[ci * 4 + 2], packed[ci * 4 + 3]);
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.p_full[t]);
    }
    // ------------------------------------------------------------------ epilogue
    const int row = tile128 * F3_BM + static_cast<int>(r);
    if (ok && nblk > 0)
      ok = mbar_wait(&ctl.pv_done[t], (nblk - 1) & 1, &ctl.abort_flag, p.status, 0xC34 + t);
    // Row sum = sum of the two halves: one fp32 exchange through the same 2 KB.
    float* lsum = reinterpret_cast<float*>(smem + F3_XCHG_OFF);
    f3_pair_sync(pair_bar);                       // nobody still reads the bf16 maxima
    lsum[(t * 2 + h) * 128 + r] = l;
    f3_pair_sync(pair_bar);
    const float l_row = lsum[(t * 2) * 128 + r] + lsum[(t * 2 + 1) * 128 + r];
    if (ok && tile128 * F3_BM < p.Sq) {
      tc_fence_after_sync();
      const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
      __nv_bfloat16* dst = p.o + ((static_cast<size_t>(batch) * p.Sq + row) * p.Hq + head) * F3_D + 64 * h;
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
int cb_attn_fwd3(const void* q, const void* k, const void* v, void* o, void* lse, int B, int Sq,
                 int Skv, int Hq, int Hkv, int q_offset, int kv_offset, int causal, float scale,
                 void* status, void* stream) {
  if (B < 1 || Sq < 1 || Skv < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0) {
    set_last_error("attention: bad shape (Hq must be a multiple of Hkv)");
    return -1;
  }
  Fa3Params p;
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
  cudaError_t e = cudaFuncSetAttribute(fa_fwd3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       F3_SMEM);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    return -1;
  }
  dim3 grid((Sq + 2 * F3_BM - 1) / (2 * F3_BM), Hq, B);
  fa_fwd3_kernel<<<grid, F3_THREADS, F3_SMEM, static_cast<cudaStream_t>(stream)>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(std::string("attention launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // extern "C"
