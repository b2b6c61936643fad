// Persistent, warp-specialised tcgen05 GEMM core for sm_100a:
//   C[M,N] = alpha * A[M,K] * B[N,K]^T     (A, B K-major; bf16 or fp8 e4m3 in, fp32
//                                           accumulation in TMEM, bf16 out)
//
// Structure (same roles as the reference's ThunderKittens GEMMs -- loader thread,
// MMA thread, epilogue warps, multi-stage TMA ring, two TMEM accumulators so the
// epilogue of tile i overlaps the main loop of tile i+1:
// datasets/example051_thunderkitten_ag_gemm_easy/nv/empty_thunderkitten_ag_gemm.cu:152-238,
// datasets/example053_thunderkitten_gemm_ar_easy/nv/empty_thunderkitten_gemm_ar.cu:84-191),
// written directly in PTX:
//   warp 0      : one elected thread issues TMA loads of A (128 x 128 B) and B (BN x 128 B)
//                 tiles into a STAGES-deep shared-memory ring (128-byte swizzle);
//   warp 1      : allocates TMEM; one elected thread issues tcgen05.mma (M=128, N=BN,
//                 K=32 bytes per instruction) and commits completion to mbarriers;
//   warp 6      : signal warp (fused kernels only): system-scope fence + flag per tile;
//   warps 2..5  : epilogue: tcgen05.ld the accumulator (warp w owns TMEM lanes
//                 32*(w%4)...), scale, convert to bf16, stage in swizzled shared memory,
//                 TMA-store 32-row x 64-column boxes.
// A `Policy` plugs in what differs between the plain GEMM and the fused
// GEMM+collective kernels: tile order, a readiness wait before a tile's A rows are
// loaded, where a finished sub-tile is stored and what is signalled afterwards.
//
// No load in this file is a cluster-multicast load.  Every wait is bounded: on a
// time-out the CTA raises its abort word, every role leaves its loop, in-flight
// copies get a grace period, TMEM is freed and the kernel returns with the
// status word set.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>

#include "../prim/tcgen05.cuh"
#include "../prim/tma.cuh"

namespace cb {

template <int BN_, int STAGES_, bool FP8_>
struct GemmCfg {
  static constexpr int BM = 128;
  static constexpr int BN = BN_;
  static constexpr bool FP8 = FP8_;
  static constexpr int BK = FP8_ ? 128 : 64;  // elements per 128-byte row
  static constexpr int MMAS_PER_STAGE = 4;    // 128 B / 32 B per instruction
  static constexpr int STAGES = STAGES_;
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_COLS = 64;                 // bf16 columns per store box (128 B)
  static constexpr int EPI_BUF_BYTES = 32 * 128;      // 32 rows x 128 B per warp and buffer
  static constexpr int EPI_BYTES = 4 * 2 * EPI_BUF_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int THREADS = 224;  // producer, MMA, 4 epilogue warps, signal warp
  static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "BN in {64,128,192,256}");
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS >= 32 && TMEM_COLS <= 512,
                "TMEM columns must be a power of two");
  static_assert(SMEM_BYTES <= 232448, "over the 227 KB shared-memory limit");
};

struct GemmShape {
  int M, N, K;
  int num_m_blocks, num_n_blocks, num_k_blocks;
  float alpha;
};

// Grouped rasterisation: consecutive tiles share a panel of up to `group` row
// blocks so the CTAs that run together reuse A and B tiles out of L2.
__device__ __forceinline__ void raster_tile(int tile, int num_m, int num_n, int group, int* m_blk,
                                            int* n_blk) {
  const int per_group = group * num_n;
  const int g = tile / per_group;
  const int first_m = g * group;
  const int gsize = (num_m - first_m) < group ? (num_m - first_m) : group;
  const int in_g = tile - g * per_group;
  *m_blk = first_m + in_g % gsize;
  *n_blk = in_g / gsize;
}

// Shared-memory control block placed after the tile ring.
template <int STAGES>
struct GemmCtl {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t sig_full[8];   // epilogue warps -> signal warp: a tile's stores were issued
  uint64_t sig_empty[8];  // signal warp -> epilogue warps: slot may be reused
  uint32_t tmem_base;
  int abort_flag;
};

// The three role loops.  `P` is the policy's parameter block.
//
// Policy interface (all static, all __device__):
//   int  num_tiles(const P&)
//   void tile_coord(const P&, int tile, int* m_blk, int* n_blk)
//   const CUtensorMap* map_a(const P&, int m_blk), map_b(const P&)
//   int  a_row(const P&, int m_blk)            row coordinate of the A tile in map_a
//   bool wait_a_ready(const P&, int m_blk, volatile int* abort)   (producer thread only)
//   static constexpr bool kDirect            false: TMA-store epilogue (store_box);
//                                              true: load/store epilogue (direct_targets)
//   void store_box(const P&, int m_blk, int n_blk, int row_in_tile, int col_in_tile,
//                  const void* smem_box)       issued by one lane; must issue exactly one
//                                              bulk-group worth of stores (commit is done here)
//   void direct_targets(const P&, int m_blk, int n_blk, DirectTargets*)
//   int  b_row(const P&, int m_blk, int n_blk)  row coordinate of the B tile in map_b
//   direct policies also: kSignalPerTile (signal warp raises a flag per tile) and
//   kScatterRows (+ uint8_t* row_base(const P&, int m_blk, int row): per-row destinations)
//   void tile_done(const P&, int m_blk, int n_blk, int quadrant)  after the quadrant's boxes
//                                              were issued (one lane)
template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_producer(const P& p, const GemmShape& g, uint8_t* ring,
                                              GemmCtl<Cfg::STAGES>* ctl, uint32_t* status,
                                              int cta, int num_ctas) {
  uint32_t stage = 0, phase = 0;
  const int ntiles = Policy::num_tiles(p);
  for (int tile = cta; tile < ntiles; tile += num_ctas) {
    int m_blk, n_blk;
    Policy::tile_coord(p, tile, &m_blk, &n_blk);
    if (!Policy::wait_a_ready(p, m_blk, &ctl->abort_flag)) return;
    const CUtensorMap* ma = Policy::map_a(p, m_blk);
    const CUtensorMap* mb = Policy::map_b(p);
    const int arow = Policy::a_row(p, m_blk);
    for (int kb = 0; kb < g.num_k_blocks; ++kb) {
      if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, &ctl->abort_flag, status, 0x100 + stage))
        return;
      uint8_t* sa = ring + stage * Cfg::STAGE_BYTES;
      uint8_t* sb = sa + Cfg::A_BYTES;
      mbar_arrive_expect_tx(&ctl->full[stage], Cfg::STAGE_BYTES);
      tma_load_2d(sa, ma, kb * Cfg::BK, arow, &ctl->full[stage]);
      tma_load_2d(sb, mb, kb * Cfg::BK, Policy::b_row(p, m_blk, n_blk), &ctl->full[stage]);
      if (++stage == Cfg::STAGES) {
        stage = 0;
        phase ^= 1u;
      }
    }
  }
}

template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_mma(const P& p, const GemmShape& g, uint8_t* ring,
                                         GemmCtl<Cfg::STAGES>* ctl, uint32_t* status, int cta,
                                         int num_ctas, uint32_t tmem_base) {
  constexpr uint32_t idesc = make_idesc(Cfg::BM, Cfg::BN, Cfg::FP8 ? 0u : 1u);
  uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
  const int ntiles = Policy::num_tiles(p);
  for (int tile = cta; tile < ntiles; tile += num_ctas) {
    if (!mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1u, &ctl->abort_flag, status, 0x200 + acc))
      return;
    tc_fence_after_sync();
    const uint32_t d_tmem = tmem_base + acc * Cfg::BN;
    for (int kb = 0; kb < g.num_k_blocks; ++kb) {
      if (!mbar_wait(&ctl->full[stage], phase, &ctl->abort_flag, status, 0x300 + stage)) return;
      tc_fence_after_sync();
      const uint32_t sa = smem_u32(ring + stage * Cfg::STAGE_BYTES);
      const uint64_t a_desc = make_sw128_kmajor_desc(sa);
      const uint64_t b_desc = make_sw128_kmajor_desc(sa + Cfg::A_BYTES);
#pragma unroll
      for (int k = 0; k < Cfg::MMAS_PER_STAGE; ++k) {
        // 32 bytes along K per instruction: +2 in the descriptor's 16-byte address units.
        const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
        if constexpr (Cfg::FP8)
          mma_fp8_ss(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, accum);
        else
          mma_bf16_ss(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, accum);
      }
      mma_commit(&ctl->empty[stage]);  // ring slot is free once these MMAs have read it
      if (++stage == Cfg::STAGES) {
        stage = 0;
        phase ^= 1u;
      }
    }
    mma_commit(&ctl->tmem_full[acc]);  // accumulator complete
    acc ^= 1u;
    if (acc == 0u) acc_phase ^= 1u;
  }
}

// fp32 accumulator row (64 columns) -> bf16, written into a [32 rows][128 B]
// buffer with the 128-byte swizzle the TMA store expects (16-byte chunk index
// XOR row%8).
__device__ __forceinline__ void epi_write_row_swizzled(uint8_t* buf, uint32_t lane,
                                                       const uint32_t (&r0)[32],
                                                       const uint32_t (&r1)[32], float alpha) {
  uint8_t* row = buf + lane * 128u;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = c * 8 + j * 2;
      const float x = __uint_as_float(col < 32 ? r0[col] : r1[col - 32]) * alpha;
      const float y = __uint_as_float(col + 1 < 32 ? r0[col + 1] : r1[col + 1 - 32]) * alpha;
      __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    const uint32_t phys = (static_cast<uint32_t>(c) ^ (lane & 7u)) * 16u;
    *reinterpret_cast<uint4*>(row + phys) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// Where a "direct" policy wants a finished tile: up to 8 destinations (peer or
// local global memory) that all receive the same data with plain 16-byte stores.
struct DirectTargets {
  uint8_t* base[8];    // address of (tile row 0, tile column 0) at each destination
  int n;               // destinations
  long long ld_bytes;  // row pitch at the destination
  int rows, cols;      // valid rows / columns of this tile (columns a multiple of 8)
};

// fp32 accumulator row (64 columns) -> bf16 into a [32 rows][256 B] buffer; chunk
// index (0..15) XOR row%8 keeps both the row-wise writes and the row-contiguous
// reads below free of bank conflicts.
__device__ __forceinline__ void epi_write_row_256(uint8_t* buf, uint32_t lane, int half_chunk,
                                                  const uint32_t (&r0)[32],
                                                  const uint32_t (&r1)[32], float alpha) {
  uint8_t* row = buf + lane * 256u;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = c * 8 + j * 2;
      const float x = __uint_as_float(col < 32 ? r0[col] : r1[col - 32]) * alpha;
      const float y = __uint_as_float(col + 1 < 32 ? r0[col + 1] : r1[col + 1 - 32]) * alpha;
      __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    const uint32_t idx = static_cast<uint32_t>(half_chunk * 8 + c);
    const uint32_t phys = (idx ^ (lane & 7u)) * 16u;
    *reinterpret_cast<uint4*>(row + phys) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// Epilogue for policies with `kDirect`: accumulator -> bf16 -> shared memory
// (transposition) -> row-contiguous 16-byte global stores, 256 bytes per row and
// half-warp.  Used where the destination is another GPU: load/store traffic
// keeps NVLink busy with few SMs, and no TMA store sits between data and flag.
template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_epilogue_direct(const P& p, const GemmShape& g,
                                                     uint8_t* epi_smem,
                                                     GemmCtl<Cfg::STAGES>* ctl, uint32_t* status,
                                                     int cta, int num_ctas, uint32_t tmem_base,
                                                     uint32_t warp, uint32_t lane) {
  const uint32_t q = warp & 3u;
  uint8_t* buf = epi_smem + q * (2 * Cfg::EPI_BUF_BYTES);  // 8 KB: 32 rows x 256 B
  uint32_t acc = 0, acc_phase = 0, seq = 0;
  const int ntiles = Policy::num_tiles(p);
  constexpr int HALVES = (Cfg::BN + 127) / 128;
  for (int tile = cta; tile < ntiles; tile += num_ctas) {
    int m_blk, n_blk;
    Policy::tile_coord(p, tile, &m_blk, &n_blk);
    DirectTargets tg;
    Policy::direct_targets(p, m_blk, n_blk, &tg);
    if (!mbar_wait(&ctl->tmem_full[acc], acc_phase, &ctl->abort_flag, status, 0x400 + acc)) return;
    tc_fence_after_sync();
#pragma unroll 1
    for (int h = 0; h < HALVES; ++h) {
      constexpr int CH = Cfg::BN >= 128 ? 2 : 1;  // 64-column chunks per half
#pragma unroll
      for (int cc = 0; cc < CH; ++cc) {
        const uint32_t taddr =
            tmem_base + ((q * 32u) << 16) + acc * Cfg::BN + (h * CH + cc) * Cfg::EPI_COLS;
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(taddr, r0);
        tmem_ld_32x32(taddr + 32u, r1);
        tmem_wait_ld();
        if (h == HALVES - 1 && cc == CH - 1) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->tmem_empty[acc]);
        }
        epi_write_row_256(buf, lane, cc, r0, r1, g.alpha);
      }
      __syncwarp();
      // Half-warp per row: 16 lanes x 16 B = 256 B (128 bf16 columns; 64 when BN == 64).
      const uint32_t idx = lane & 15u;
      const int col = h * 128 + static_cast<int>(idx) * 8;
      const bool col_ok = (static_cast<int>(idx) < CH * 8) && col < tg.cols;
#pragma unroll 4
      for (int i = 0; i < 16; ++i) {
        const uint32_t r = 2u * i + (lane >> 4);
        const int row = static_cast<int>(q * 32u + r);
        const uint4 v = *reinterpret_cast<const uint4*>(buf + r * 256u + ((idx ^ (r & 7u)) * 16u));
        if constexpr (Policy::kScatterRows) {
          // Every output row has its own destination (MoE combine): look it up.
          uint8_t* rb = col_ok ? Policy::row_base(p, m_blk, row) : nullptr;
          if (rb != nullptr) st_sys_v4(rb + (static_cast<long long>(n_blk) * Cfg::BN + col) * 2ll, v);
        } else if (col_ok && row < tg.rows) {
          const long long off = row * tg.ld_bytes + col * 2ll;
          for (int d = 0; d < tg.n; ++d) st_sys_v4(tg.base[d] + off, v);
        }
      }
      __syncwarp();
    }
    // Hand the tile to the signal warp: it runs the (slow, ~20 us under store traffic)
    // system-scope fence and raises the flag while these warps go on with the next tile.
    __syncwarp();
    if (Policy::kSignalPerTile && lane == 0) {
      const uint32_t slot = seq & 7u;
      if (!mbar_wait(&ctl->sig_empty[slot], ((seq >> 3) & 1u) ^ 1u, &ctl->abort_flag, status,
                     0x800 + slot))
        return;
      mbar_arrive(&ctl->sig_full[slot]);
    }
    ++seq;
    acc ^= 1u;
    if (acc == 0u) acc_phase ^= 1u;
  }
}

// Signal warp of a direct policy: for the tiles of this CTA, wait until the four
// epilogue warps have issued a tile's stores, make them visible system-wide,
// signal.  A system-scope fence under store traffic costs tens of microseconds,
// so it runs here, off the epilogue's path, and one fence covers every tile that
// became ready while the previous fence was draining (up to 4).  Cumulativity
// covers the epilogue warps' stores: their lanes synchronised with the arriving
// lane, which synchronised with this thread through the mbarrier.
template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_signal(const P& p, GemmCtl<Cfg::STAGES>* ctl,
                                            uint32_t* status, int cta, int num_ctas) {
  uint32_t seq = 0;
  const int ntiles = Policy::num_tiles(p);
  int pend_m[4], pend_n[4];
  int npend = 0;
  int tile = cta;
  while (tile < ntiles || npend > 0) {
    if (tile < ntiles && npend < 4) {
      const uint32_t slot = seq & 7u;
      const uint32_t par = (seq >> 3) & 1u;
      bool ready = mbar_try_wait(&ctl->sig_full[slot], par);
      if (!ready && npend == 0) {
        if (!mbar_wait(&ctl->sig_full[slot], par, &ctl->abort_flag, status, 0x900 + slot)) return;
        ready = true;
      }
      if (ready) {
        mbar_arrive(&ctl->sig_empty[slot]);
        Policy::tile_coord(p, tile, &pend_m[npend], &pend_n[npend]);
        ++npend;
        tile += num_ctas;
        ++seq;
        continue;
      }
    }
    fence_acq_rel_sys();  // release; a sequentially-consistent fence costs far more here
    for (int i = 0; i < npend; ++i) Policy::tile_done(p, pend_m[i], pend_n[i], 0);
    npend = 0;
  }
}

// A policy may declare `static constexpr bool kGated = true`: every BN-wide accumulator tile then
// holds BN/2 "gate" columns followed by BN/2 "up" columns of the same output columns (the
// weight rows are interleaved that way by the caller), and the TMA-store epilogue writes
// silu(gate) * up - BN/2 output columns per tile - instead of the raw accumulator, so the
// activation never makes a round trip through HBM.
template <class Policy>
__host__ __device__ constexpr bool policy_gated() {
  if constexpr (requires { Policy::kGated; }) {
    return Policy::kGated;
  } else {
    return false;
  }
}

// acc[i] <- silu(alpha * acc[i]) * (alpha * up[i]), fp32 in the accumulator's bit pattern.
__device__ __forceinline__ void epi_gate_32(uint32_t (&acc)[32], const uint32_t (&up)[32],
                                            float alpha) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float gv = __uint_as_float(acc[i]) * alpha;
    const float uv = __uint_as_float(up[i]) * alpha;
    acc[i] = __float_as_uint(gv / (1.f + __expf(-gv)) * uv);
  }
}

template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_epilogue_tma(const P& p, const GemmShape& g,
                                                  uint8_t* epi_smem, GemmCtl<Cfg::STAGES>* ctl,
                                                  uint32_t* status, int cta, int num_ctas,
                                                  uint32_t tmem_base, uint32_t warp,
                                                  uint32_t lane) {
  const uint32_t q = warp & 3u;  // TMEM lane quadrant this warp may read
  uint8_t* bufs = epi_smem + q * (2 * Cfg::EPI_BUF_BYTES);
  uint32_t acc = 0, acc_phase = 0, buf = 0;
  const int ntiles = Policy::num_tiles(p);
  for (int tile = cta; tile < ntiles; tile += num_ctas) {
    int m_blk, n_blk;
    Policy::tile_coord(p, tile, &m_blk, &n_blk);
    if (!mbar_wait(&ctl->tmem_full[acc], acc_phase, &ctl->abort_flag, status, 0x400 + acc)) return;
    tc_fence_after_sync();
    constexpr bool kGated = policy_gated<Policy>();
    constexpr int kBoxes = Cfg::BN / Cfg::EPI_COLS / (kGated ? 2 : 1);  // store boxes per tile
#pragma unroll 1
    for (int c = 0; c < kBoxes; ++c) {
      const uint32_t taddr = tmem_base + ((q * 32u) << 16) + acc * Cfg::BN + c * Cfg::EPI_COLS;
      uint32_t r0[32], r1[32];
      if constexpr (kGated) {
        uint32_t up[32];
        tmem_ld_32x32(taddr, r0);
        tmem_ld_32x32(taddr + Cfg::BN / 2, up);
        tmem_wait_ld();
        epi_gate_32(r0, up, g.alpha);
        tmem_ld_32x32(taddr + 32u, r1);
        tmem_ld_32x32(taddr + Cfg::BN / 2 + 32u, up);
        tmem_wait_ld();
        epi_gate_32(r1, up, g.alpha);
      } else {
        tmem_ld_32x32(taddr, r0);
        tmem_ld_32x32(taddr + 32u, r1);
        tmem_wait_ld();
      }
      if (c == kBoxes - 1) {
        // Last read of this accumulator: hand it back to the MMA thread.
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->tmem_empty[acc]);
      }
      // The buffer we are about to fill was read by the store issued two boxes ago.
      if (lane == 0) bulk_wait_read<1>();
      __syncwarp();
      uint8_t* b = bufs + buf * Cfg::EPI_BUF_BYTES;
      epi_write_row_swizzled(b, lane, r0, r1, kGated ? 1.0f : g.alpha);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        Policy::store_box(p, m_blk, n_blk, static_cast<int>(q * 32u), c * Cfg::EPI_COLS, b);
        bulk_commit();
      }
      buf ^= 1u;
    }
    if (lane == 0) Policy::tile_done(p, m_blk, n_blk, static_cast<int>(q));
    acc ^= 1u;
    if (acc == 0u) acc_phase ^= 1u;
  }
  if (lane == 0) bulk_wait_all<0>();
}

template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_epilogue(const P& p, const GemmShape& g, uint8_t* epi_smem,
                                              GemmCtl<Cfg::STAGES>* ctl, uint32_t* status,
                                              int cta, int num_ctas, uint32_t tmem_base,
                                              uint32_t warp, uint32_t lane) {
  if constexpr (Policy::kDirect) {
    gemm_epilogue_direct<Cfg, Policy>(p, g, epi_smem, ctl, status, cta, num_ctas, tmem_base, warp,
                                      lane);
  } else {
    gemm_epilogue_tma<Cfg, Policy>(p, g, epi_smem, ctl, status, cta, num_ctas, tmem_base, warp,
                                   lane);
  }
}

// Common prologue / epilogue of every kernel built on this core.
template <class Cfg>
__device__ __forceinline__ uint8_t* gemm_smem_base(uint8_t* raw) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023u) & ~uintptr_t(1023));
}

template <class Cfg>
__device__ __forceinline__ uint32_t gemm_setup(GemmCtl<Cfg::STAGES>* ctl, uint32_t warp) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&ctl->tmem_full[a], 1);
      mbar_init(&ctl->tmem_empty[a], 4);  // one arrival per epilogue warp
    }
    for (int i = 0; i < 8; ++i) {
      mbar_init(&ctl->sig_full[i], 4);
      mbar_init(&ctl->sig_empty[i], 1);
    }
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  return *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
}

template <class Cfg>
__device__ __forceinline__ void gemm_teardown(GemmCtl<Cfg::STAGES>* ctl, uint32_t warp,
                                              uint32_t tmem_base) {
  tc_fence_before_sync();
  __syncthreads();
  if (*reinterpret_cast<volatile int*>(&ctl->abort_flag) != 0) {
    // Some wait gave up: loads may still be landing in this CTA's shared memory.
    // Give them a bounded grace period before the CTA (and its memory) goes away.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace cb

namespace cb {

// Whole-CTA body: set-up, the three roles, tear-down.  `cta` / `num_ctas`
// number the CTAs that share the tile list (fused kernels reserve some CTAs of
// the grid for communication, and rank emulation splits the grid per rank).
template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_cta_main(const P& p, const GemmShape& g, uint32_t* status,
                                              int cta, int num_ctas, uint8_t* smem_raw) {
  uint8_t* smem = gemm_smem_base<Cfg>(smem_raw);
  uint8_t* ring = smem;
  uint8_t* epi = smem + Cfg::STAGES * Cfg::STAGE_BYTES;
  __shared__ GemmCtl<Cfg::STAGES> ctl;
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t tmem_base = gemm_setup<Cfg>(&ctl, warp);
  if (warp == 0) {
    if (lane == 0) gemm_producer<Cfg, Policy>(p, g, ring, &ctl, status, cta, num_ctas);
  } else if (warp == 1) {
    if (lane == 0) gemm_mma<Cfg, Policy>(p, g, ring, &ctl, status, cta, num_ctas, tmem_base);
  } else if (warp < 6) {
    gemm_epilogue<Cfg, Policy>(p, g, epi, &ctl, status, cta, num_ctas, tmem_base, warp, lane);
  } else {
    if constexpr (Policy::kDirect && Policy::kSignalPerTile) {
      if (lane == 0) gemm_signal<Cfg, Policy>(p, &ctl, status, cta, num_ctas);
    }
  }
  __syncwarp();
  gemm_teardown<Cfg>(&ctl, warp, tmem_base);
}

}  // namespace cb
