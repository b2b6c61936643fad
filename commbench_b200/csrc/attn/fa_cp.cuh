// Context-parallel flash-attention forward: ONE kernel that pulls the remote key/value
// shards into local memory with a few communication CTAs while the other CTAs attend to the
// shards that are already there, and carries the running (max, sum, O) of a query tile across
// ALL shards in registers / tensor memory - no partial results, no merge launches.
//
// The attention math is the kernel of fa_fwd4.cu (two 128-row query tiles per CTA, a softmax
// warp-group per tile, S / P / O in tensor memory, K ring of 3 and V ring of 2).  What is
// generalised here:
//   * keys and values are a list of SEGMENTS of one local buffer (row range, global position of
//     the first key, optional "ready" counter).  Ring attention lists the shards in ring
//     order - own shard first, then rank-1, rank-2, ... - Ulysses lists the sequence in order;
//     the producer warp waits for a segment's counter before its first TMA load from it;
//   * queries are a list of QUERY SEGMENTS (tensor map, row range, global position, output
//     tensor): the two zig-zag halves of a ring shard, or - for Ulysses - the W sequence shards,
//     whose Q tiles are fetched straight from their owners' memory with plain (non-multicast)
//     TMA loads and whose O rows are stored straight into their owners' output tensors;
//   * registers are moved from the four utility warps (producer, MMA issuer, two idle) to
//     the eight softmax warps with setmaxnreg (72 / 216 per thread), which keeps a 128-column row
//     of scores in registers without spills, and every `kPoly`-th pair of exponentials is
//     computed on the FMA pipe (a cubic after a round-to-nearest split) instead of the SFU,
//     which otherwise is as busy as the tensor pipe;
//   * CTAs draw tickets: the first `num_comm` tickets copy the list of 2-D pieces
//     (peer -> local, 16-byte loads and stores), bumping each piece's counter when done; the
//     others take (query tile pair, head, batch) items, heaviest first.
// No CTA waits for another GPU inside this kernel: remote data is pulled, and the cross-GPU
// barriers that say "shards are published" / "shards may be overwritten" bracket the launch.
//
// The reference's context-parallel examples are the communication halves only - the K/V ring
// rotation of datasets/example057_thunderkitten_ring_attn_easy/nv/empty_thunderkitten_ring_attn.cu:97-134
// (stage schedule :336-379) and the four Ulysses all-to-alls of
// datasets/example058_thunderkitten_ulysses_attn_easy/nv/empty_thunderkitten_ulysses_attn.cu:59-120,
// :330-359 - with the attention itself left out.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>

#include "../prim/tcgen05.cuh"
#include "../prim/tma.cuh"
#include "fa_cp_types.h"

namespace cb {

struct CpCtl {
  uint64_t q_full;
  uint64_t k_full[CP_KST], k_empty[CP_KST];
  uint64_t v_full[CP_VST], v_empty[CP_VST];
  uint64_t s_full[2], p_full[2], pv_done[2];  // per query tile
  uint32_t tmem_base;
  int abort_flag;
  int ticket;
};

__device__ __forceinline__ uint64_t cp_mnmajor_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(CP_SUB >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__device__ __forceinline__ float cp_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint64_t cp_pack_u(uint32_t lo, uint32_t hi) {
  return static_cast<uint64_t>(lo) | (static_cast<uint64_t>(hi) << 32);
}
__device__ __forceinline__ uint64_t cp_pack(float lo, float hi) {
  return cp_pack_u(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ uint64_t cp_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t cp_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float cp_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Walks the key blocks that a query tile pair attends to, segment by segment.  Every role of a
// CTA runs its own copy and sees the same sequence.  Both tiles of the pair visit the same
// blocks: a block that lies wholly in the future of the first tile (at most one per item, the
// diagonal block of the second tile) is visited with everything masked.
struct CpBlockIter {
  int seg, i, n;  // current segment, block inside it, visible blocks of that segment
  __device__ __forceinline__ static int visible(const FaCpParams& p, int s, int q_last) {
    const CpSeg& g = p.seg[s];
    int n = (g.nkeys + CP_BN - 1) / CP_BN;
    if (p.causal) {
      const int lim = q_last - g.kpos0;
      if (lim < 0) return 0;
      const int c = lim / CP_BN + 1;
      if (c < n) n = c;
    }
    return n;
  }
  __device__ __forceinline__ void start(const FaCpParams& p, int q_last) {
    seg = -1;
    i = 0;
    n = 0;
    advance(p, q_last);
  }
  __device__ __forceinline__ void advance(const FaCpParams& p, int q_last) {
    for (++seg; seg < p.nseg; ++seg) {
      n = visible(p, seg, q_last);
      if (n > 0) break;
    }
    i = 0;
  }
  __device__ __forceinline__ void next(const FaCpParams& p, int q_last) {
    if (++i >= n) advance(p, q_last);
  }
  __device__ __forceinline__ static int total(const FaCpParams& p, int q_last) {
    int t = 0;
    for (int s = 0; s < p.nseg; ++s) t += visible(p, s, q_last);
    return t;
  }
};

// Communication CTA `c` of `p.num_comm`: its share of every piece, in list order.
__device__ __forceinline__ void cp_comm_cta(const FaCpParams& p, int c) {
  const int T = blockDim.x;
  for (int ci = 0; ci < p.ncopy; ++ci) {
    const CpCopy cp = p.copies[ci];
    const int vpr = cp.row_bytes >> 4;
    const long long total = static_cast<long long>(cp.nrows) * vpr;
    // vector -> (row, column); one-row pieces and power-of-two rows avoid the division
    const bool pow2 = (vpr & (vpr - 1)) == 0;
    const int sh = pow2 ? __ffs(vpr) - 1 : 0;
    auto locate = [&](long long w, long long* so, long long* dn) {
      long long row, col;
      if (cp.nrows == 1) {
        row = 0;
        col = w;
      } else if (pow2) {
        row = w >> sh;
        col = w & (vpr - 1);
      } else {
        row = w / vpr;
        col = w - row * vpr;
      }
      *so = row * cp.src_pitch + col * 16;
      *dn = row * cp.dst_pitch + col * 16;
    };
    long long v = static_cast<long long>(c) * T + threadIdx.x;
    const long long step = static_cast<long long>(p.num_comm) * T;
    for (; v + 7 * step < total; v += 8 * step) {
      uint4 x[8];
      long long dn[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        long long so;
        locate(v + u * step, &so, &dn[u]);
        x[u] = ld_sys_v4(cp.src + so);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) st_v4(cp.dst + dn[u], x[u]);
    }
    for (; v < total; v += step) {
      long long so, dn;
      locate(v, &so, &dn);
      st_v4(cp.dst + dn, ld_sys_v4(cp.src + so));
    }
    __syncthreads();
    if (threadIdx.x == 0 && cp.flag >= 0) red_release_gpu_add(p.flags + cp.flag, 1u);
  }
}

template <int N>
__device__ __forceinline__ void cp_reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void cp_reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// kPoly: every kPoly-th pair of keys takes its exponential from the FMA pipe (0: none).
template <int kPoly>
__global__ void __launch_bounds__(CP_THREADS, 1) fa_cp_kernel(const __grid_constant__ FaCpParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem =
      reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + 2 * CP_TILE;
  uint8_t* sV = sK + CP_KST * CP_TILE;
  __shared__ CpCtl ctl;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;

  // Tickets only where communication CTAs must be the first to run; a launch without them
  // (plain local attention) takes its item from the block index.
  int ticket = static_cast<int>(blockIdx.x);
  if (p.sched != nullptr) {
    if (threadIdx.x == 0) ctl.ticket = static_cast<int>(atomicAdd(&p.sched[0], 1u));
    __syncthreads();
    ticket = ctl.ticket;
  }
  bool attend = false;
  int qs_i = 0, pair = 0, head = 0, batch = 0;
  if (ticket < p.num_comm) {
    cp_comm_cta(p, ticket);
  } else {
    // item -> (query segment, tile pair inside it, head, batch); pairs run from the end of a
    // segment to its start (under a causal mask the late rows are the long items)
    int item = ticket - p.num_comm;
    const int per_pair = p.heads * p.B;
    int gp = item / per_pair;
    const int rem = item - gp * per_pair;
    head = rem % p.heads;
    batch = rem / p.heads;
    for (qs_i = 0; qs_i < p.nqseg; ++qs_i) {
      const int np = (p.qseg[qs_i].nrows + 2 * CP_BM - 1) / (2 * CP_BM);
      if (gp < np) {
        pair = np - 1 - gp;
        attend = true;
        break;
      }
      gp -= np;
    }
  }

  if (attend) {
    const CpQSeg qs = p.qseg[qs_i];
    const int q_first = qs.qpos0 + pair * 2 * CP_BM;          // position of row 0 of tile 0
    int rows_here = qs.nrows - pair * 2 * CP_BM;              // valid query rows of this pair
    if (rows_here > 2 * CP_BM) rows_here = 2 * CP_BM;
    const int q_last = q_first + rows_here - 1;
    const int nblk = CpBlockIter::total(p, q_last);
    const int kv_head = head / p.kv_group;

    if (threadIdx.x == 0) {
      mbar_init(&ctl.q_full, 1);
      for (int i = 0; i < CP_KST; ++i) {
        mbar_init(&ctl.k_full[i], 1);
        mbar_init(&ctl.k_empty[i], 1);
      }
      for (int i = 0; i < CP_VST; ++i) {
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
    // tile t: S (fp32, 128 columns; its first 64 columns hold P as bf16 pairs after the
    // softmax) at column 256 t, O at column 256 t + 128.

    // 128 x 72 + 256 x 216 registers = 64,512 of the SM's 65,536.
    if (warp < 4) {
    cp_reg_dec<72>();
    if (warp == 0) {
      if (lane == 0 && nblk > 0) {
        // ---------------------------------------------------------------- producer
        const CUtensorMap* tmq = qs.map < 0 ? &p.tm_q_local : p.tm_q_arr + qs.map;
        mbar_arrive_expect_tx(&ctl.q_full, 2 * CP_TILE);
        const int qrow = batch * p.q_bstride + qs.row0 + pair * 2 * CP_BM;
        for (int t = 0; t < 2; ++t) {
          tma_load_3d(sQ + t * CP_TILE, tmq, 0, p.q_head0 + head, qrow + t * CP_BM, &ctl.q_full);
          tma_load_3d(sQ + t * CP_TILE + CP_SUB, tmq, 64, p.q_head0 + head, qrow + t * CP_BM,
                      &ctl.q_full);
        }
        CpBlockIter ik, iv;
        ik.start(p, q_last);
        iv.start(p, q_last);
        int jk = 0, jv = 0, ready_seg = -1;
        bool ok = true;
        uint32_t idle = 0;
        uint64_t t0 = 0;
        while (ok && (jk < nblk || jv < nblk)) {
          bool progress = false;
          if (jk < nblk) {
            const int s = jk % CP_KST, use = jk / CP_KST;
            if (use == 0 || mbar_try_wait(&ctl.k_empty[s], (use - 1) & 1)) {
              // First block of a segment that is still being pulled: wait for its counter.
              // K and V of a segment arrive under the same counter.
              if (ik.seg != ready_seg) {
                const CpSeg& g = p.seg[ik.seg];
                if (g.flag >= 0) {
                  if (!wait_flag_ge_gpu(p.flags + g.flag, p.flag_target, p.timeout_ns, p.status,
                                        40, static_cast<uint32_t>(ik.seg))) {
                    ctl.abort_flag = 1;
                    ok = false;
                    break;
                  }
                  fence_proxy_async();  // the rows were written with ordinary stores
                }
                ready_seg = ik.seg;
              }
              const int krow = batch * p.kv_bstride + p.seg[ik.seg].row0 + ik.i * CP_BN;
              mbar_arrive_expect_tx(&ctl.k_full[s], CP_TILE);
              tma_load_3d(sK + s * CP_TILE, &p.tm_k, 0, kv_head, krow, &ctl.k_full[s]);
              tma_load_3d(sK + s * CP_TILE + CP_SUB, &p.tm_k, 64, kv_head, krow, &ctl.k_full[s]);
              ++jk;
              ik.next(p, q_last);
              progress = true;
            }
          }
          if (jv < nblk && jv < jk) {
            const int s = jv % CP_VST, use = jv / CP_VST;
            if (use == 0 || mbar_try_wait(&ctl.v_empty[s], (use - 1) & 1)) {
              const int vrow = batch * p.kv_bstride + p.seg[iv.seg].row0 + iv.i * CP_BN;
              mbar_arrive_expect_tx(&ctl.v_full[s], CP_TILE);
              tma_load_3d(sV + s * CP_TILE, &p.tm_v, 0, kv_head, vrow, &ctl.v_full[s]);
              tma_load_3d(sV + s * CP_TILE + CP_SUB, &p.tm_v, 64, kv_head, vrow, &ctl.v_full[s]);
              ++jv;
              iv.next(p, q_last);
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
              report_status(p.status, CB_TIMEOUT_MBARRIER, 0, 0xE00);
              break;
            }
          }
        }
      }
    } else if (warp == 1) {
      if (nblk > 0) {
        // --------------------------------------------------------------------- MMA
        // The whole warp walks the schedule and waits; one elected lane issues.
        constexpr uint32_t idesc_s = make_idesc(128, 128, 1u);
        constexpr uint32_t idesc_pv = make_idesc(128, 128, 1u) | (1u << 16);  // V is MN-major
        const uint64_t q_desc0 = make_sw128_kmajor_desc(smem_u32(sQ));
        const uint64_t k_desc0 = make_sw128_kmajor_desc(smem_u32(sK));
        const uint64_t v_desc0 = cp_mnmajor_desc(smem_u32(sV));
        constexpr uint64_t kTileStep = static_cast<uint64_t>(CP_TILE >> 4);
        constexpr uint64_t kSubStep = static_cast<uint64_t>(CP_SUB >> 4);
        auto wait_all = [&](uint64_t* bar, uint32_t parity, uint32_t detail) -> bool {
          const bool w = mbar_wait(bar, parity, &ctl.abort_flag, p.status, detail);
          return __all_sync(0xffffffffu, w ? 1 : 0) != 0;
        };
        bool ok = wait_all(&ctl.q_full, 0, 0xE10);
        auto issue_qk = [&](int t, int j) -> bool {
          const int s = j % CP_KST;
          if (!wait_all(&ctl.k_full[s], (j / CP_KST) & 1, 0xE11)) return false;
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
          const int s = j % CP_VST;
          if (!wait_all(&ctl.p_full[t], j & 1, 0xE20 + t)) return false;
          if (!wait_all(&ctl.v_full[s], (j / CP_VST) & 1, 0xE22)) return false;
          tc_fence_after_sync();
          if (elect_one()) {
            const uint64_t va = v_desc0 + s * kTileStep;
            const uint32_t d = tmem + 256u * t + 128u;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              mma_bf16_ts(d, tmem + 256u * t + 8u * kk, va + kk * (2048u >> 4), idesc_pv,
                          (j > 0 || kk > 0) ? 1u : 0u);
            mma_commit(&ctl.pv_done[t]);
          }
          __syncwarp();
          return true;
        };
        for (int t = 0; ok && t < 2; ++t) ok = issue_qk(t, 0);
        if (ok && elect_one()) mma_commit(&ctl.k_empty[0]);
        __syncwarp();
        for (int j = 0; ok && j < nblk; ++j) {
          for (int t = 0; ok && t < 2; ++t) {
            ok = issue_pv(t, j);
            if (ok && j + 1 < nblk) ok = issue_qk(t, j + 1);
          }
          if (!ok) break;
          if (elect_one()) {
            mma_commit(&ctl.v_empty[j % CP_VST]);
            if (j + 1 < nblk) mma_commit(&ctl.k_empty[(j + 1) % CP_KST]);
          }
          __syncwarp();
        }
      }
    }
    } else {
      cp_reg_inc<216>();
      // ------------------------------------------------------------------- softmax
      const int t = warp >= 8 ? 1 : 0;
      const uint32_t q = warp & 3u;
      const uint32_t r = q * 32u + lane;
      const uint32_t lane_addr = (q * 32u) << 16;
      const uint32_t tS = tmem + 256u * t + lane_addr;
      const uint32_t tO = tS + 128u;
      const int row_in_seg = pair * 2 * CP_BM + t * CP_BM + static_cast<int>(r);
      const int tile_first = q_first + t * CP_BM;     // position of row 0 of this tile
      const int q_pos = tile_first + static_cast<int>(r);
      float m_ref = -INFINITY, l = 0.f;
      bool ok = true;
      CpBlockIter it;
      it.start(p, q_last);
      for (int j = 0; ok && j < nblk; ++j) {
        if (!mbar_wait(&ctl.s_full[t], j & 1, &ctl.abort_flag, p.status, 0xE30 + t)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        uint32_t s[128];
        tmem_ld_32x32_at(tS, &s[0]);
        tmem_ld_32x32_at(tS + 32u, &s[32]);
        tmem_ld_32x32_at(tS + 64u, &s[64]);
        tmem_ld_32x32_at(tS + 96u, &s[96]);
        tmem_wait_ld();

        const CpSeg& g = p.seg[it.seg];
        const int key0 = g.kpos0 + it.i * CP_BN;
        const int kv_left = g.nkeys - it.i * CP_BN;
        const bool need_mask = kv_left < CP_BN || (p.causal && key0 + CP_BN - 1 > tile_first);
        it.next(p, q_last);
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (!(i < kv_left && (!p.causal || key0 + i <= q_pos))) s[i] = 0xff800000u;  // -inf
        }
        float mx8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          mx8[i] = fmaxf(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1]));
#pragma unroll
        for (int i = 16; i < 128; i += 2)
          mx8[(i >> 1) & 7] =
              cp_max3(mx8[(i >> 1) & 7], __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
        const float mx_all =
            cp_max3(fmaxf(cp_max3(mx8[0], mx8[1], mx8[2]), cp_max3(mx8[3], mx8[4], mx8[5])),
                    mx8[6], mx8[7]);
        const float mx_s = mx_all * p.scale_log2;
        const bool grow =
            mx_s > m_ref + CP_RESCALE_THRESHOLD || (m_ref == -INFINITY && mx_s > -INFINITY);
        const bool any_grow = __any_sync(0xffffffffu, grow);
        if (any_grow) {
          const float m_new = fmaxf(m_ref, mx_s);
          const float alpha = m_ref == -INFINITY ? 0.f : cp_ex2(m_ref - m_new);
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
        const uint64_t scale2 = cp_pack(p.scale_log2, p.scale_log2), negm2 = cp_pack(-m_use, -m_use);
        uint64_t sum4[4] = {0ull, 0ull, 0ull, 0ull};
        // The bf16 pairs go back into s[0..63]: element i is only written after s[2i], s[2i+1]
        // have been consumed.
#pragma unroll
        for (int i = 0; i < 128; i += 2) {
          const uint64_t y = cp_fma2(cp_pack_u(s[i], s[i + 1]), scale2, negm2);
          float p0, p1;
          if (kPoly > 0 && !need_mask && ((i >> 1) % (kPoly > 0 ? kPoly : 1)) == kPoly - 1) {
            // 2^x on the FMA pipe: nearest-integer split with the 1.5 * 2^23 trick, a cubic on
            // the fraction in [-0.5, 0.5] (relative error 7.5e-5, below bf16 rounding), the
            // exponent added as an integer; inputs clamped to -126 so it cannot wrap.  Masked
            // blocks keep the SFU everywhere: -inf must give an exact zero.
            const float x0 = fmaxf(__uint_as_float(static_cast<uint32_t>(y)), -126.f);
            const float x1 = fmaxf(__uint_as_float(static_cast<uint32_t>(y >> 32)), -126.f);
            const uint64_t xx = cp_pack(x0, x1);
            const uint64_t rr = cp_add2(xx, cp_pack(12582912.f, 12582912.f));
            const uint64_t xf = cp_add2(rr, cp_pack(-12582912.f, -12582912.f));
            const uint64_t fr = cp_fma2(xf, cp_pack(-1.f, -1.f), xx);
            uint64_t qq = cp_fma2(fr, cp_pack(0.05517116f, 0.05517116f), cp_pack(0.24261014f, 0.24261014f));
            qq = cp_fma2(qq, fr, cp_pack(0.69326097f, 0.69326097f));
            qq = cp_fma2(qq, fr, cp_pack(0.99992812f, 0.99992812f));
            p0 = __uint_as_float(static_cast<uint32_t>(qq) + (static_cast<uint32_t>(rr) << 23));
            p1 = __uint_as_float(static_cast<uint32_t>(qq >> 32) + (static_cast<uint32_t>(rr >> 32) << 23));
          } else {
            p0 = cp_ex2(__uint_as_float(static_cast<uint32_t>(y)));
            p1 = cp_ex2(__uint_as_float(static_cast<uint32_t>(y >> 32)));
          }
          sum4[(i >> 1) & 3] = cp_add2(sum4[(i >> 1) & 3], cp_pack(p0, p1));
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          s[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
        }
        {
          const uint64_t a = cp_add2(cp_add2(sum4[0], sum4[1]), cp_add2(sum4[2], sum4[3]));
          l += __uint_as_float(static_cast<uint32_t>(a)) + __uint_as_float(static_cast<uint32_t>(a >> 32));
        }
        // P_t(j): row r = lane r, keys 2c and 2c+1 in column c.
        tmem_st_32x32_at(tS, &s[0]);
        tmem_st_32x32_at(tS + 32u, &s[32]);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.p_full[t]);
      }
      // ------------------------------------------------------------------ epilogue
      if (ok && nblk > 0)
        ok = mbar_wait(&ctl.pv_done[t], (nblk - 1) & 1, &ctl.abort_flag, p.status, 0xE34 + t);
      // Tile-uniform condition: the tensor-memory loads below are warp-collective; rows past
      // the end of the segment are only kept from being stored.
      if (ok && pair * 2 * CP_BM + t * CP_BM < qs.nrows) {
        const bool row_ok = row_in_seg < qs.nrows;
        tc_fence_after_sync();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int orow = qs.row0 + row_in_seg;
        __nv_bfloat16* dst =
            p.o[qs.out] + ((static_cast<size_t>(batch) * p.o_rows[qs.out] + orow) * p.o_heads +
                           p.o_head0 + head) * CP_D;
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
          if (row_ok) {
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
        if (row_ok && p.lse[qs.out] != nullptr)
          p.lse[qs.out][(static_cast<size_t>(batch) * p.o_heads + p.o_head0 + head) *
                            p.o_rows[qs.out] + orow] =
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

  // Last CTA out re-arms the ticket counter for the next launch.
  __syncthreads();
  if (threadIdx.x == 0 && p.sched != nullptr) {
    __threadfence();
    if (atomicAdd(&p.sched[1], 1u) == gridDim.x - 1u) {
      p.sched[0] = 0u;
      p.sched[1] = 0u;
      __threadfence();
    }
  }
}

}  // namespace cb
