// Flash-attention forward, second design: two query tiles of 128 rows per CTA, one softmax
// warp-group per tile, O accumulated in tensor memory.
//
//   warp 0      TMA producer: both Q tiles once, then K (two stages) and V (one stage) per
//               block of 128 keys; K and V are issued as soon as their buffer is free,
//               whichever comes first
//   warp 1      MMA issuer; per key block j:  S_0 = Q_0 K_j^T, S_1 = Q_1 K_j^T, then
//               O_0 += P_0(j-1) V_{j-1}, O_1 += P_1(j-1) V_{j-1}  (accumulating in TMEM)
//   warps 2-5   softmax of tile 0, warps 6-9 softmax of tile 1: one query row per thread.
//               The 128 scores of the row are read from TMEM ONCE (and the S buffer is handed
//               back to the MMA warp right away), max / exp2 / row sum run with eight
//               independent accumulators, P goes to shared memory as the bf16 K-major
//               operand of the second MMA.
//
// O is only rescaled when the running maximum grew by more than 2^8 since the reference
// maximum was last changed (the exponentials then stay below 2^8 = 256, exact in the final
// O / l); with that the rescale - a TMEM read-modify-write of the row - is rare after the
// first blocks.  While one tile's warps run their softmax, the tensor core works on the
// other tile.
//
// Output: normalised O of this key/value chunk plus the row-wise log-sum-exp, as the first
// design (fa_fwd.cu), so ring steps can be merged exactly.  Every wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include <string>

#include "../gemm/tmap_host.h"
#include "../prim/tcgen05.cuh"
#include "../prim/tma.cuh"
#include "../symm/driver_api.h"

namespace cb {

static constexpr int F2_BM = 128;     // rows per query tile
static constexpr int F2_BN = 128;     // keys per block
static constexpr int F2_D = 128;      // head dim
static constexpr int F2_SUB = 16384;  // bytes of one [128 x 64] bf16 sub-tile
static constexpr int F2_TILE = 2 * F2_SUB;
// Q: 2 tiles, K: 2 stages, V: 1 stage, P: 2 tiles.
static constexpr int F2_SMEM = 2 * F2_TILE + 2 * F2_TILE + F2_TILE + 2 * F2_TILE + 1024;
static constexpr int F2_THREADS = 320;
static constexpr float F2_RESCALE_THRESHOLD = 8.f;  // log2 units

struct Fa2Params {
  CUtensorMap tm_q;  // 3-D {D, Hq, B*Sq}, box {64, 1, 128}
  CUtensorMap tm_k;  // 3-D {D, Hkv, B*Skv}
  CUtensorMap tm_v;
  __nv_bfloat16* o;  // [B, Sq, Hq, D]
  float* lse;        // [B, Hq, Sq]
  int B, Sq, Skv, Hq, Hkv;
  int q_offset, kv_offset;
  int causal;
  float scale_log2;
  uint32_t* status;
};

struct Fa2Ctl {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2];
  uint64_t v_full, v_empty;
  uint64_t s_full[2], s_empty[2];   // per query tile
  uint64_t p_full[2], pv_done[2];   // per query tile
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint64_t f2_mnmajor_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(F2_SUB >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__device__ __forceinline__ float f2_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Blackwell packed fp32 pairs and three-input max.
__device__ __forceinline__ uint64_t f2_pack_u(uint32_t lo, uint32_t hi) {
  return static_cast<uint64_t>(lo) | (static_cast<uint64_t>(hi) << 32);
}
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  return f2_pack_u(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ uint64_t f2_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float f2_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Key blocks that the 128-row tile `tile128` can see.
__device__ __forceinline__ int f2_num_blocks(const Fa2Params& p, int tile128) {
  if (tile128 * F2_BM >= p.Sq) return 0;
  int nblk = (p.Skv + F2_BN - 1) / F2_BN;
  if (p.causal) {
    const int last_q = p.q_offset + (tile128 + 1) * F2_BM - 1;
    const int lim = last_q - p.kv_offset;
    if (lim < 0) return 0;
    const int c = lim / F2_BN + 1;
    if (c < nblk) nblk = c;
  }
  return nblk;
}

// kPolyEvery: every kPolyEvery-th pair of keys computes 2^x on the FMA pipe (0: none).
template <int kPolyEvery>
__global__ void __launch_bounds__(F2_THREADS, 1)
    fa_fwd2_kernel(const __grid_constant__ Fa2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem =
      reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                 // [tile][2 sub-tiles]
  uint8_t* sK = sQ + 2 * F2_TILE;     // [stage][2 sub-tiles]
  uint8_t* sV = sK + 2 * F2_TILE;     // one stage
  uint8_t* sP = sV + F2_TILE;         // [tile][2 sub-tiles]
  __shared__ Fa2Ctl ctl;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  // Long (late) query tiles first: they carry the most key blocks under a causal mask.
  const int q_pair = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int nblk0 = f2_num_blocks(p, 2 * q_pair), nblk1 = f2_num_blocks(p, 2 * q_pair + 1);
  const int nblk_max = nblk0 > nblk1 ? nblk0 : nblk1;

  if (threadIdx.x == 0) {
    mbar_init(&ctl.q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl.k_full[i], 1);
      mbar_init(&ctl.k_empty[i], 1);
      mbar_init(&ctl.s_full[i], 1);
      mbar_init(&ctl.s_empty[i], 4);
      mbar_init(&ctl.p_full[i], 4);
      mbar_init(&ctl.pv_done[i], 1);
    }
    mbar_init(&ctl.v_full, 1);
    mbar_init(&ctl.v_empty, 1);
    ctl.abort_flag = 0;
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
  // tile t: S at column 256 t, O at column 256 t + 128

  if (warp == 0) {
    if (lane == 0 && nblk_max > 0) {
      // ---------------------------------------------------------------- producer
      mbar_arrive_expect_tx(&ctl.q_full, 2 * F2_TILE);
      const int qrow = batch * p.Sq + q_pair * 2 * F2_BM;
      for (int t = 0; t < 2; ++t) {
        tma_load_3d(sQ + t * F2_TILE, &p.tm_q, 0, head, qrow + t * F2_BM, &ctl.q_full);
        tma_load_3d(sQ + t * F2_TILE + F2_SUB, &p.tm_q, 64, head, qrow + t * F2_BM, &ctl.q_full);
      }
      int jk = 0, jv = 0;
      uint32_t idle = 0;
      uint64_t t0 = 0;
      while (jk < nblk_max || jv < nblk_max) {
        bool progress = false;
        if (jk < nblk_max) {
          const int s = jk & 1;
          if (jk < 2 || mbar_try_wait(&ctl.k_empty[s], ((jk >> 1) - 1) & 1)) {
            const int krow = batch * p.Skv + jk * F2_BN;
            mbar_arrive_expect_tx(&ctl.k_full[s], F2_TILE);
            tma_load_3d(sK + s * F2_TILE, &p.tm_k, 0, kv_head, krow, &ctl.k_full[s]);
            tma_load_3d(sK + s * F2_TILE + F2_SUB, &p.tm_k, 64, kv_head, krow, &ctl.k_full[s]);
            ++jk;
            progress = true;
          }
        }
        if (jv < nblk_max && jv < jk) {
          if (jv < 1 || mbar_try_wait(&ctl.v_empty, (jv - 1) & 1)) {
            const int vrow = batch * p.Skv + jv * F2_BN;
            mbar_arrive_expect_tx(&ctl.v_full, F2_TILE);
            tma_load_3d(sV, &p.tm_v, 0, kv_head, vrow, &ctl.v_full);
            tma_load_3d(sV + F2_SUB, &p.tm_v, 64, kv_head, vrow, &ctl.v_full);
            ++jv;
            progress = true;
          }
        }
        if (progress) {
          idle = 0;
          continue;
        }
        // Bounded: give up when somebody else did, or after 4 s without progress.
        if ((++idle & 255u) == 0u) {
          if (*reinterpret_cast<volatile int*>(&ctl.abort_flag) != 0) break;
          const uint64_t now = globaltimer_ns();
          if (t0 == 0 || idle == 256u) t0 = now;
          if (now - t0 > CB_MBAR_TIMEOUT_NS) {
            ctl.abort_flag = 1;
            report_status(p.status, CB_TIMEOUT_MBARRIER, 0, 0xB00);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nblk_max > 0) {
      // --------------------------------------------------------------------- MMA
      constexpr uint32_t idesc_s = make_idesc(128, 128, 1u);
      constexpr uint32_t idesc_pv = make_idesc(128, 128, 1u) | (1u << 16);  // B is MN-major
      const int nb[2] = {nblk0, nblk1};
      bool ok = mbar_wait(&ctl.q_full, 0, &ctl.abort_flag, p.status, 0xB10);
      auto issue_pv = [&](int t, int j) -> bool {
        if (!mbar_wait(&ctl.p_full[t], j & 1, &ctl.abort_flag, p.status, 0xB20 + t)) return false;
        if (!mbar_wait(&ctl.v_full, j & 1, &ctl.abort_flag, p.status, 0xB22)) return false;
        tc_fence_after_sync();
        const uint32_t pa = smem_u32(sP + t * F2_TILE), va = smem_u32(sV);
        const uint32_t d = tmem + 256u * t + 128u;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a_desc = make_sw128_kmajor_desc(pa + (kk >> 2) * F2_SUB) + 2u * (kk & 3);
          const uint64_t b_desc = f2_mnmajor_desc(va + kk * 2048);
          mma_bf16_ss(d, a_desc, b_desc, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        }
        mma_commit(&ctl.pv_done[t]);
        return true;
      };
      for (int j = 0; ok && j < nblk_max; ++j) {
        const int s = j & 1;
        ok = mbar_wait(&ctl.k_full[s], (j >> 1) & 1, &ctl.abort_flag, p.status, 0xB11);
        for (int t = 0; ok && t < 2; ++t) {
          if (j >= nb[t]) continue;
          ok = mbar_wait(&ctl.s_empty[t], (j & 1) ^ 1u, &ctl.abort_flag, p.status, 0xB12 + t);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t qa = smem_u32(sQ + t * F2_TILE), ka = smem_u32(sK + s * F2_TILE);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t a_desc = make_sw128_kmajor_desc(qa + (kk >> 2) * F2_SUB) + 2u * (kk & 3);
            const uint64_t b_desc = make_sw128_kmajor_desc(ka + (kk >> 2) * F2_SUB) + 2u * (kk & 3);
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
  } else {
    // ------------------------------------------------------------------- softmax
    const int t = warp >= 6 ? 1 : 0;           // query tile of this warp-group
    const int nblk = t ? nblk1 : nblk0;
    const uint32_t q = warp & 3u;              // TMEM lane quadrant this warp may touch
    const uint32_t r = q * 32u + lane;         // row inside the tile
    const uint32_t lane_addr = (q * 32u) << 16;
    const uint32_t tS = tmem + 256u * t + lane_addr;
    const uint32_t tO = tS + 128u;
    const int tile128 = 2 * q_pair + t;
    const int q_pos = p.q_offset + tile128 * F2_BM + static_cast<int>(r);
    uint8_t* sPt = sP + t * F2_TILE;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; ok && j < nblk; ++j) {
      if (!mbar_wait(&ctl.s_full[t], j & 1, &ctl.abort_flag, p.status, 0xB30 + t)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t s[128];
      tmem_ld_32x32_at(tS, &s[0]);
      tmem_ld_32x32_at(tS + 32u, &s[32]);
      tmem_ld_32x32_at(tS + 64u, &s[64]);
      tmem_ld_32x32_at(tS + 96u, &s[96]);
      tmem_wait_ld();
      // The scores are in registers: the MMA warp may overwrite S with the next block.
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.s_empty[t]);

      const int key0 = p.kv_offset + j * F2_BN;
      const int kv_left = p.Skv - j * F2_BN;
      const bool need_mask = kv_left < F2_BN ||
                             (p.causal && key0 + F2_BN - 1 > p.q_offset + tile128 * F2_BM);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (!(i < kv_left && (!p.causal || key0 + i <= q_pos))) s[i] = 0xff800000u;  // -inf
      }
      // Row maximum: three-input max, eight independent chains.
      float mx8[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx8[i] = fmaxf(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1]));
#pragma unroll
      for (int i = 16; i < 128; i += 2)
        mx8[(i >> 1) & 7] = f2_max3(mx8[(i >> 1) & 7], __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
      const float mx = fmaxf(f2_max3(mx8[0], mx8[1], mx8[2]), f2_max3(mx8[3], mx8[4], mx8[5]));
      const float mx_all = f2_max3(mx, mx8[6], mx8[7]);
      const float mx_s = mx_all * p.scale_log2;  // scale > 0; -inf stays -inf
      const bool grow = mx_s > m_ref + F2_RESCALE_THRESHOLD || (m_ref == -INFINITY && mx_s > -INFINITY);
      const bool any_grow = __any_sync(0xffffffffu, grow);
      float alpha = 1.f;
      if (any_grow) {
        const float m_new = fmaxf(m_ref, mx_s);
        alpha = m_ref == -INFINITY ? 0.f : f2_ex2(m_ref - m_new);
        m_ref = m_new;
        l *= alpha;
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      const float neg_m = -m_use;
      // p = 2^(s * scale - m): the multiply-add and the row sum run as packed two-wide fp32
      // operations (one instruction per pair of keys), the exponential on the SFU.
      const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2), negm2 = f2_pack(neg_m, neg_m);
      uint64_t sum4[4] = {0ull, 0ull, 0ull, 0ull};
      uint32_t packed[64];
      if (need_mask) {
        // Masked entries are -inf and must come out as exact zeros: SFU path for all.
#pragma unroll
        for (int i = 0; i < 128; i += 2) {
          const uint64_t y = f2_fma2(f2_pack_u(s[i], s[i + 1]), scale2, negm2);
          const float p0 = f2_ex2(__uint_as_float(static_cast<uint32_t>(y)));
          const float p1 = f2_ex2(__uint_as_float(static_cast<uint32_t>(y >> 32)));
          sum4[(i >> 1) & 3] = f2_add2(sum4[(i >> 1) & 3], f2_pack(p0, p1));
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
        }
      } else {
        // The SFU (16 exponentials per clock and SM) is the busiest pipe here, so every
        // kPolyEvery-th pair of keys takes its 2^x from the FMA pipe instead: round to the
        // nearest integer with the 1.5*2^23 trick, a cubic on the fraction in [-0.5, 0.5]
        // (relative error 7.5e-5, far below the bf16 rounding of P), exponent added as an
        // integer.  Inputs are clamped to -126 so the exponent cannot wrap.
#pragma unroll
        for (int i = 0; i < 128; i += 2) {
          const uint64_t y = f2_fma2(f2_pack_u(s[i], s[i + 1]), scale2, negm2);
          float p0, p1;
          if (kPolyEvery > 0 && ((i >> 1) % (kPolyEvery > 0 ? kPolyEvery : 1)) == kPolyEvery - 1) {
            const float x0 = fmaxf(__uint_as_float(static_cast<uint32_t>(y)), -126.f);
            const float x1 = fmaxf(__uint_as_float(static_cast<uint32_t>(y >> 32)), -126.f);
            const uint64_t xx = f2_pack(x0, x1);
            const uint64_t magic = f2_pack(12582912.f, 12582912.f);
            const uint64_t r = f2_add2(xx, magic);
            const uint64_t xf = f2_add2(r, f2_pack(-12582912.f, -12582912.f));
            const uint64_t fr = f2_fma2(xf, f2_pack(-1.f, -1.f), xx);
            uint64_t q = f2_fma2(fr, f2_pack(0.05517116f, 0.05517116f), f2_pack(0.24261014f, 0.24261014f));
            q = f2_fma2(q, fr, f2_pack(0.69326097f, 0.69326097f));
            q = f2_fma2(q, fr, f2_pack(0.99992812f, 0.99992812f));
            p0 = __uint_as_float(static_cast<uint32_t>(q) + (static_cast<uint32_t>(r) << 23));
            p1 = __uint_as_float(static_cast<uint32_t>(q >> 32) + (static_cast<uint32_t>(r >> 32) << 23));
          } else {
            p0 = f2_ex2(__uint_as_float(static_cast<uint32_t>(y)));
            p1 = f2_ex2(__uint_as_float(static_cast<uint32_t>(y >> 32)));
          }
          sum4[(i >> 1) & 3] = f2_add2(sum4[(i >> 1) & 3], f2_pack(p0, p1));
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      {
        const uint64_t a = f2_add2(f2_add2(sum4[0], sum4[1]), f2_add2(sum4[2], sum4[3]));
        l += __uint_as_float(static_cast<uint32_t>(a)) + __uint_as_float(static_cast<uint32_t>(a >> 32));
      }

      // P(j-1) V(j-1) must have completed: it read the P buffer and wrote O.
      if (!mbar_wait(&ctl.pv_done[t], (j & 1) ^ 1u, &ctl.abort_flag, p.status, 0xB32 + t)) { ok = false; break; }
      if (any_grow && j > 0) {
        tc_fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
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
      for (int ch = 0; ch < 16; ++ch) {
        const uint32_t sub = ch >> 3, ci = ch & 7u;
        uint8_t* dst = sPt + sub * F2_SUB + r * 128u + ((ci ^ (r & 7u)) * 16u);
        *reinterpret_cast<uint4*>(dst) = make_uint4(packed[ch * 4], packed[ch * 4 + 1],
                                                    packed[ch * 4 + 2], packed[ch * 4 + 3]);
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.p_full[t]);
    }
    // ------------------------------------------------------------------ epilogue
    const int row = tile128 * F2_BM + static_cast<int>(r);
    if (ok && nblk > 0)
      ok = mbar_wait(&ctl.pv_done[t], (nblk - 1) & 1, &ctl.abort_flag, p.status, 0xB34 + t);
    if (ok && tile128 * F2_BM < p.Sq) {
      tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.o + ((static_cast<size_t>(batch) * p.Sq + row) * p.Hq + head) * F2_D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
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
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              h[k] = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * k]) * inv,
                                           __uint_as_float(o[i + 2 * k + 1]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
          }
        }
      }
      if (row < p.Sq)
        p.lse[(static_cast<size_t>(batch) * p.Hq + head) * p.Sq + row] =
            l > 0.f ? (m_ref * 0.6931471805599453f + logf(l)) : -INFINITY;
    }
  }
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (*reinterpret_cast<volatile int*>(&ctl.abort_flag) != 0) {
    // Some wait gave up: loads may still be landing; give them a bounded grace period.
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

// Measured on B200 (S=16384, 32 heads, causal): 882 TFLOP/s with every exponential on the SFU,
// 844 / 821 / 806 with every 4th / 3rd / 2nd pair on the FMA pipe - this kernel is bound by
// issue slots and latency in the softmax warps, not by the SFU, so the default is 0.
static int g_fa2_poly_every = 0;

extern "C" {

// How many of the exponentials leave the SFU: every n-th pair of keys (0 = none, 2, 3 or 4).
void cb_attn_set_poly_every(int n) { g_fa2_poly_every = n; }

// Same contract as cb_attn_fwd (fa_fwd.cu).
int cb_attn_fwd2(const void* q, const void* k, const void* v, void* o, void* lse, int B, int Sq,
                 int Skv, int Hq, int Hkv, int q_offset, int kv_offset, int causal, float scale,
                 void* status, void* stream) {
  if (B < 1 || Sq < 1 || Skv < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0) {
    set_last_error("attention: bad shape (Hq must be a multiple of Hkv)");
    return -1;
  }
  Fa2Params p;
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
  dim3 grid((Sq + 2 * F2_BM - 1) / (2 * F2_BM), Hq, B);
  cudaError_t e = cudaSuccess;
#define CB_FA2_LAUNCH(POLY)                                                                     \
  do {                                                                                          \
    e = cudaFuncSetAttribute(fa_fwd2_kernel<POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                             F2_SMEM);                                                          \
    if (e == cudaSuccess)                                                                       \
      fa_fwd2_kernel<POLY><<<grid, F2_THREADS, F2_SMEM, static_cast<cudaStream_t>(stream)>>>(p); \
  } while (0)
  switch (g_fa2_poly_every) {
    case 0: CB_FA2_LAUNCH(0); break;
    case 2: CB_FA2_LAUNCH(2); break;
    case 3: CB_FA2_LAUNCH(3); break;
    case 4: CB_FA2_LAUNCH(4); break;
    default: CB_FA2_LAUNCH(0); break;
  }
#undef CB_FA2_LAUNCH
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    return -1;
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(std::string("attention launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // extern "C"
