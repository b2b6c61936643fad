// Flash-attention forward, fourth design: P stays in tensor memory.
//
// As the second design (two query tiles of 128 rows per CTA, one softmax warp-group per tile,
// O accumulated in TMEM with lazy rescale, scores read once), plus:
//   * the softmax writes P (bf16) back into the first 64 columns of the tile's S region with
//     tcgen05.st, and the second MMA takes its A operand from tensor memory
//     (tcgen05.mma with [a_tmem]); P never touches shared memory, which halves the shared-memory
//     traffic of P*V and frees 64 KB;
//   * with that room K has three stages and V two, so the next block's K and V are always in
//     flight while the current block is worked on.  (With one V stage the chain
//     "P*V done -> load V -> P*V" set the pace: the same kernel with the softmax arithmetic
//     removed still ran at only 1.0 PFLOP/s.)
//
//   warp 0      TMA producer (Q tiles, K ring of 3, V ring of 2)
//   warp 1      MMA issuer; per tile t the chain is  S_t(j) -> softmax -> P_t(j) -> O_t += P_t V_j
//               -> S_t(j+1); the two tiles' chains interleave on the tensor pipe.  S_t(j+1)
//               overwrites the columns P_t(j) lived in: both MMAs come from this one thread, in
//               order, so the overwrite follows the read.
//   warps 2-5   softmax of tile 0, warps 6-9 of tile 1 (one query row per thread).
//
// The completion of S_t(j) is signalled by a commit that covers every earlier MMA of the
// issuing thread, P_t(j-1) V_{j-1} included, so a softmax warp that sees S_t(j) may rescale
// O_t and overwrite P_t without another wait.
#include <cuda.h>
#include <cuda_bf16.h>

#include <string>

#include "../gemm/tmap_host.h"
#include "../prim/tcgen05.cuh"
#include "../prim/tma.cuh"
#include "../symm/driver_api.h"

namespace cb {

static constexpr int F4_BM = 128;
static constexpr int F4_BN = 128;
static constexpr int F4_D = 128;
static constexpr int F4_SUB = 16384;
static constexpr int F4_TILE = 2 * F4_SUB;
static constexpr int F4_KST = 3, F4_VST = 2;
static constexpr int F4_SMEM = (2 + F4_KST + F4_VST) * F4_TILE + 1024;   // Q | K ring | V ring
static constexpr int F4_THREADS = 320;
static constexpr float F4_RESCALE_THRESHOLD = 8.f;

struct Fa4Params {
  CUtensorMap tm_q, tm_k, tm_v;
  __nv_bfloat16* o;
  float* lse;
  int B, Sq, Skv, Hq, Hkv;
  int q_offset, kv_offset;
  int causal;
  float scale_log2;
  uint32_t* status;
};

struct Fa4Ctl {
  uint64_t q_full;
  uint64_t k_full[F4_KST], k_empty[F4_KST];
  uint64_t v_full[F4_VST], v_empty[F4_VST];
  uint64_t s_full[2], p_full[2], pv_done[2];   // per query tile
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint64_t f4_mnmajor_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(F4_SUB >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__device__ __forceinline__ float f4_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint64_t f4_pack_u(uint32_t lo, uint32_t hi) {
  return static_cast<uint64_t>(lo) | (static_cast<uint64_t>(hi) << 32);
}
__device__ __forceinline__ uint64_t f4_pack(float lo, float hi) {
  return f4_pack_u(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ uint64_t f4_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f4_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float f4_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 32 lanes x 32 columns store from 32 consecutive elements of a larger register array.
__device__ __forceinline__ void f4_tmem_st_at(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(
          taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ int f4_num_blocks(const Fa4Params& p, int tile128) {
  if (tile128 * F4_BM >= p.Sq) return 0;
  int nblk = (p.Skv + F4_BN - 1) / F4_BN;
  if (p.causal) {
    const int last_q = p.q_offset + (tile128 + 1) * F4_BM - 1;
    const int lim = last_q - p.kv_offset;
    if (lim < 0) return 0;
    const int c = lim / F4_BN + 1;
    if (c < nblk) nblk = c;
  }
  return nblk;
}

// kPolyEvery: every kPolyEvery-th pair of keys takes its exponential from the FMA pipe (0: none).
template <int kPolyEvery>
__global__ void __launch_bounds__(F4_THREADS, 1) fa_fwd4_kernel(const __grid_constant__ Fa4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem =
      reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + 2 * F4_TILE;
  uint8_t* sV = sK + F4_KST * F4_TILE;
  __shared__ Fa4Ctl ctl;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const int q_pair = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int nblk0 = f4_num_blocks(p, 2 * q_pair), nblk1 = f4_num_blocks(p, 2 * q_pair + 1);
  const int nblk_max = nblk0 > nblk1 ? nblk0 : nblk1;

  if (threadIdx.x == 0) {
    mbar_init(&ctl.q_full, 1);
    for (int i = 0; i < F4_KST; ++i) {
      mbar_init(&ctl.k_full[i], 1);
      mbar_init(&ctl.k_empty[i], 1);
    }
    for (int i = 0; i < F4_VST; ++i) {
      mbar_init(&ctl.v_full[i], 1);
      mbar_init(&ctl.v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl.s_full[i], 1);
      mbar_init(&ctl.p_full[i], 4);
      mbar_init(&ctl.pv_done[i], 1);
    }
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
  // tile t: S (fp32, 128 columns; its first 64 columns hold P as bf16 pairs after the softmax)
  // at column 256 t, O at column 256 t + 128.

  if (warp == 0) {
    if (lane == 0 && nblk_max > 0) {
      // ---------------------------------------------------------------- producer
      mbar_arrive_expect_tx(&ctl.q_full, 2 * F4_TILE);
      const int qrow = batch * p.Sq + q_pair * 2 * F4_BM;
      for (int t = 0; t < 2; ++t) {
        tma_load_3d(sQ + t * F4_TILE, &p.tm_q, 0, head, qrow + t * F4_BM, &ctl.q_full);
        tma_load_3d(sQ + t * F4_TILE + F4_SUB, &p.tm_q, 64, head, qrow + t * F4_BM, &ctl.q_full);
      }
      int jk = 0, jv = 0;
      uint32_t idle = 0;
      uint64_t t0 = 0;
      while (jk < nblk_max || jv < nblk_max) {
        bool progress = false;
        if (jk < nblk_max) {
          const int s = jk % F4_KST, use = jk / F4_KST;
          if (use == 0 || mbar_try_wait(&ctl.k_empty[s], (use - 1) & 1)) {
            const int krow = batch * p.Skv + jk * F4_BN;
            mbar_arrive_expect_tx(&ctl.k_full[s], F4_TILE);
            tma_load_3d(sK + s * F4_TILE, &p.tm_k, 0, kv_head, krow, &ctl.k_full[s]);
            tma_load_3d(sK + s * F4_TILE + F4_SUB, &p.tm_k, 64, kv_head, krow, &ctl.k_full[s]);
            ++jk;
            progress = true;
          }
        }
        if (jv < nblk_max && jv < jk) {
          const int s = jv % F4_VST, use = jv / F4_VST;
          if (use == 0 || mbar_try_wait(&ctl.v_empty[s], (use - 1) & 1)) {
            const int vrow = batch * p.Skv + jv * F4_BN;
            mbar_arrive_expect_tx(&ctl.v_full[s], F4_TILE);
            tma_load_3d(sV + s * F4_TILE, &p.tm_v, 0, kv_head, vrow, &ctl.v_full[s]);
            tma_load_3d(sV + s * F4_TILE + F4_SUB, &p.tm_v, 64, kv_head, vrow, &ctl.v_full[s]);
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
            report_status(p.status, CB_TIMEOUT_MBARRIER, 0, 0xD00);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (nblk_max > 0) {
      // --------------------------------------------------------------------- MMA
      // The whole warp walks the schedule and waits; one elected lane issues the MMAs and
      // commits.  (Issued from inside an `if (lane == 0)` branch, a 128 x 128 x 16 MMA cost
      // ~60 cycles of issue against 64 cycles on the tensor pipe, so the issuing thread, not the
      // pipe or the softmax, set the pace.)
      constexpr uint32_t idesc_s = make_idesc(128, 128, 1u);
      constexpr uint32_t idesc_pv = make_idesc(128, 128, 1u) | (1u << 16);  // B (= V) is MN-major
      const int nb[2] = {nblk0, nblk1};
      const uint64_t q_desc0 = make_sw128_kmajor_desc(smem_u32(sQ));
      const uint64_t k_desc0 = make_sw128_kmajor_desc(smem_u32(sK));
      const uint64_t v_desc0 = f4_mnmajor_desc(smem_u32(sV));
      constexpr uint64_t kTileStep = static_cast<uint64_t>(F4_TILE >> 4);
      constexpr uint64_t kSubStep = static_cast<uint64_t>(F4_SUB >> 4);
      auto wait_all = [&](uint64_t* bar, uint32_t parity, uint32_t detail) -> bool {
        const bool w = mbar_wait(bar, parity, &ctl.abort_flag, p.status, detail);
        return __all_sync(0xffffffffu, w ? 1 : 0) != 0;
      };
      bool ok = wait_all(&ctl.q_full, 0, 0xD10);
      auto issue_qk = [&](int t, int j) -> bool {
        const int s = j % F4_KST;
        if (!wait_all(&ctl.k_full[s], (j / F4_KST) & 1, 0xD11)) return false;
        tc_fence_after_sync();
        if (elect_one()) {
          const uint64_t qa = q_desc0 + t * kTileStep, ka = k_desc0 + s * kTileStep;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t off = (kk >> 2) * kSubStep + 2u * (kk & 3);
            mma_bf16_ss(tmem + 256u * t, qa + off, ka + off, idesc_s, kk > 0 ? 1u : 0u);
          }
          mma_commit(&ctl.s_full[t]);
        }
        __syncwarp();
        return true;
      };
      auto issue_pv = [&](int t, int j) -> bool {
        const int s = j % F4_VST;
        if (!wait_all(&ctl.p_full[t], j & 1, 0xD20 + t)) return false;
        if (!wait_all(&ctl.v_full[s], (j / F4_VST) & 1, 0xD22)) return false;
        tc_fence_after_sync();
        if (elect_one()) {
          const uint64_t va = v_desc0 + s * kTileStep;
          const uint32_t d = tmem + 256u * t + 128u;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            // A = P_t from tensor memory: 16 keys = 8 columns of bf16 pairs per step.
            mma_bf16_ts(d, tmem + 256u * t + 8u * kk, va + kk * (2048u >> 4), idesc_pv,
                        (j > 0 || kk > 0) ? 1u : 0u);
          }
          mma_commit(&ctl.pv_done[t]);
        }
        __syncwarp();
        return true;
      };
      // prologue: S_t(0) of both tiles
      for (int t = 0; ok && t < 2; ++t)
        if (nb[t] > 0) ok = issue_qk(t, 0);
      if (ok && elect_one()) mma_commit(&ctl.k_empty[0]);
      __syncwarp();
      for (int j = 0; ok && j < nblk_max; ++j) {
        for (int t = 0; ok && t < 2; ++t) {
          if (j >= nb[t]) continue;
          ok = issue_pv(t, j);
          if (ok && j + 1 < nb[t]) ok = issue_qk(t, j + 1);
        }
        if (!ok) break;
        if (elect_one()) {
          mma_commit(&ctl.v_empty[j % F4_VST]);
          if (j + 1 < nblk_max) mma_commit(&ctl.k_empty[(j + 1) % F4_KST]);
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------- softmax
    const int t = warp >= 6 ? 1 : 0;
    const int nblk = t ? nblk1 : nblk0;
    const uint32_t q = warp & 3u;
    const uint32_t r = q * 32u + lane;
    const uint32_t lane_addr = (q * 32u) << 16;
    const uint32_t tS = tmem + 256u * t + lane_addr;
    const uint32_t tO = tS + 128u;
    const int tile128 = 2 * q_pair + t;
    const int q_pos = p.q_offset + tile128 * F4_BM + static_cast<int>(r);
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; ok && j < nblk; ++j) {
      if (!mbar_wait(&ctl.s_full[t], j & 1, &ctl.abort_flag, p.status, 0xD30 + t)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t s[128];
      tmem_ld_32x32_at(tS, &s[0]);
      tmem_ld_32x32_at(tS + 32u, &s[32]);
      tmem_ld_32x32_at(tS + 64u, &s[64]);
      tmem_ld_32x32_at(tS + 96u, &s[96]);
      tmem_wait_ld();

      const int key0 = p.kv_offset + j * F4_BN;
      const int kv_left = p.Skv - j * F4_BN;
      const bool need_mask = kv_left < F4_BN ||
                             (p.causal && key0 + F4_BN - 1 > p.q_offset + tile128 * F4_BM);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (!(i < kv_left && (!p.causal || key0 + i <= q_pos))) s[i] = 0xff800000u;  // -inf
      }
      float mx8[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx8[i] = fmaxf(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1]));
#pragma unroll
      for (int i = 16; i < 128; i += 2)
        mx8[(i >> 1) & 7] = f4_max3(mx8[(i >> 1) & 7], __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
      const float mx_all = f4_max3(fmaxf(f4_max3(mx8[0], mx8[1], mx8[2]), f4_max3(mx8[3], mx8[4], mx8[5])),
                                   mx8[6], mx8[7]);
      const float mx_s = mx_all * p.scale_log2;
      const bool grow = mx_s > m_ref + F4_RESCALE_THRESHOLD || (m_ref == -INFINITY && mx_s > -INFINITY);
      const bool any_grow = __any_sync(0xffffffffu, grow);
      float alpha = 1.f;
      if (any_grow) {
        const float m_new = fmaxf(m_ref, mx_s);
        alpha = m_ref == -INFINITY ? 0.f : f4_ex2(m_ref - m_new);
        m_ref = m_new;
        l *= alpha;
        if (j > 0) {
          // S_t(j) complete implies P_t(j-1) V_{j-1} complete: O_t is stable.
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tO + c * 32u, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tO + c * 32u, o);
          }
        }
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      const uint64_t scale2 = f4_pack(p.scale_log2, p.scale_log2), negm2 = f4_pack(-m_use, -m_use);
      uint64_t sum4[4] = {0ull, 0ull, 0ull, 0ull};
      // The bf16 pairs go back into s[0..63]: element i is only written after s[2i], s[2i+1]
      // have been consumed.
#pragma unroll
      for (int i = 0; i < 128; i += 2) {
        const uint64_t y = f4_fma2(f4_pack_u(s[i], s[i + 1]), scale2, negm2);
        float p0, p1;
        if (kPolyEvery > 0 && !need_mask && ((i >> 1) % (kPolyEvery > 0 ? kPolyEvery : 1)) == kPolyEvery - 1) {
          // 2^x on the FMA pipe for this pair (the SFU sets the latency of a block's softmax,
          // which sits on the per-tile critical path S -> P -> O): nearest-integer split with the
          // 1.5 * 2^23 trick, a cubic on the fraction in [-0.5, 0.5] (relative error 7.5e-5), the
          // exponent added as an integer; inputs clamped to -126 so the exponent cannot wrap.
          // Masked blocks keep the SFU everywhere: -inf must give an exact zero.
          const float x0 = fmaxf(__uint_as_float(static_cast<uint32_t>(y)), -126.f);
          const float x1 = fmaxf(__uint_as_float(static_cast<uint32_t>(y >> 32)), -126.f);
          const uint64_t xx = f4_pack(x0, x1);
          const uint64_t rr = f4_add2(xx, f4_pack(12582912.f, 12582912.f));
          const uint64_t xf = f4_add2(rr, f4_pack(-12582912.f, -12582912.f));
          const uint64_t fr = f4_fma2(xf, f4_pack(-1.f, -1.f), xx);
          uint64_t qq = f4_fma2(fr, f4_pack(0.05517116f, 0.05517116f), f4_pack(0.24261014f, 0.24261014f));
          qq = f4_fma2(qq, fr, f4_pack(0.69326097f, 0.69326097f));
          qq = f4_fma2(qq, fr, f4_pack(0.99992812f, 0.99992812f));
          p0 = __uint_as_float(static_cast<uint32_t>(qq) + (static_cast<uint32_t>(rr) << 23));
          p1 = __uint_as_float(static_cast<uint32_t>(qq >> 32) + (static_cast<uint32_t>(rr >> 32) << 23));
        } else {
          p0 = f4_ex2(__uint_as_float(static_cast<uint32_t>(y)));
          p1 = f4_ex2(__uint_as_float(static_cast<uint32_t>(y >> 32)));
        }
        sum4[(i >> 1) & 3] = f4_add2(sum4[(i >> 1) & 3], f4_pack(p0, p1));
        __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
        s[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
      }
      {
        const uint64_t a = f4_add2(f4_add2(sum4[0], sum4[1]), f4_add2(sum4[2], sum4[3]));
        l += __uint_as_float(static_cast<uint32_t>(a)) + __uint_as_float(static_cast<uint32_t>(a >> 32));
      }
      // P_t(j): row r = lane r, keys 2c and 2c+1 in column c.
      f4_tmem_st_at(tS, &s[0]);
      f4_tmem_st_at(tS + 32u, &s[32]);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.p_full[t]);
    }
    // ------------------------------------------------------------------ epilogue
    const int row = tile128 * F4_BM + static_cast<int>(r);
    if (ok && nblk > 0)
      ok = mbar_wait(&ctl.pv_done[t], (nblk - 1) & 1, &ctl.abort_flag, p.status, 0xD34 + t);
    if (ok && tile128 * F4_BM < p.Sq) {
      tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.o + ((static_cast<size_t>(batch) * p.Sq + row) * p.Hq + head) * F4_D;
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
            __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              hh[k] = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * k]) * inv,
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

static int g_fa4_poly_every = 0;

extern "C" {

// Every n-th pair of keys computes its exponential on the FMA pipe (0 = none, 2, 3 or 4).
void cb_attn4_set_poly_every(int n) { g_fa4_poly_every = n; }

// Same contract as cb_attn_fwd (fa_fwd.cu).
int cb_attn_fwd4(const void* q, const void* k, const void* v, void* o, void* lse, int B, int Sq,
                 int Skv, int Hq, int Hkv, int q_offset, int kv_offset, int causal, float scale,
                 void* status, void* stream) {
  if (B < 1 || Sq < 1 || Skv < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0) {
    set_last_error("attention: bad shape (Hq must be a multiple of Hkv)");
    return -1;
  }
  Fa4Params p;
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
  dim3 grid((Sq + 2 * F4_BM - 1) / (2 * F4_BM), Hq, B);
  cudaError_t e = cudaSuccess;
#define CB_FA4_LAUNCH(POLY)                                                                     \
  do {                                                                                          \
    e = cudaFuncSetAttribute(fa_fwd4_kernel<POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                             F4_SMEM);                                                          \
    if (e == cudaSuccess)                                                                       \
      fa_fwd4_kernel<POLY><<<grid, F4_THREADS, F4_SMEM, static_cast<cudaStream_t>(stream)>>>(p); \
  } while (0)
  switch (g_fa4_poly_every) {
    case 2: CB_FA4_LAUNCH(2); break;
    case 3: CB_FA4_LAUNCH(3); break;
    case 4: CB_FA4_LAUNCH(4); break;
    default: CB_FA4_LAUNCH(0); break;
  }
#undef CB_FA4_LAUNCH
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
