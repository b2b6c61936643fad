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
//   warp 0      : one elected lane issues TMA loads of A (128 x 128 B) and B (BN x 128 B)
//                 tiles into a STAGES-deep shared-memory ring (128-byte swizzle);
//   warp 1      : allocates TMEM; one elected lane issues tcgen05.mma (M=128, N=BN,
//                 K=32 bytes per instruction) and commits completion to mbarriers;
//   warp 6      : signal warp (fused kernels only): system-scope fence + flag per tile;
//   warps 2..5  : epilogue: tcgen05.ld the accumulator (warp w owns TMEM lanes
//                 32*(w%4)...), scale, convert to bf16, stage in swizzled shared memory,
//                 TMA-store 32-row x 64-column boxes.
// A `Policy` plugs in what differs between the plain GEMM and the fused
// GEMM+collective kernels: tile order, a readiness wait before a tile's A rows are
// loaded, where a finished sub-tile is stored and what is signalled afterwards.
//
//
// CTA pairs (`PAIR_ = 2`, launched as clusters of two): the two CTAs share one
// 256 x BN tile the way the reference's `CLUSTER_SIZE = 2` GEMMs do
// (datasets/example051_thunderkitten_ag_gemm_easy/nv/empty_thunderkitten_ag_gemm.cu:73,86-99).
// CTA r of the pair loads rows 128r.. of the A tile and rows (BN/2)r.. of the B
// tile with its own plain TMA loads, whose bytes are counted on the even CTA's
// mbarrier; the even CTA's MMA thread issues `tcgen05.mma.cta_group::2`
// (M = 256), which makes each tensor core read its own A half and both B
// halves, so the B traffic out of shared memory halves and the ring gets
// deeper; completion is committed to the barriers of both CTAs; each CTA drains
// its own 128 accumulator rows.  `Cfg::BM` is the height of a tile (128 or 256)
// and is what policies count row blocks in.
//
// Block-scaled fp8 (`BS_ = true`): A carries one fp32 scale per row and 128 K-elements, B one
// per 128 x 128 block (the "1x128 / 128x128" recipe).  One ring stage is one 128-wide K block;
// the MMA thread starts a FRESH accumulator for every K block, alternating between the two
// TMEM buffers, and commits it; eight epilogue warps (two per TMEM lane quadrant, 128 columns
// each) read the partial sum, multiply it by a_scale[row, kb] * b_scale[n block, kb] and add it
// to a running fp32 sum kept in registers - the promotion step that fp8 tensor cores need for
// long K anyway - while the tensor core works on the next K block.  The quantised operands go
// straight from memory into the MMA; nothing is expanded to bf16.
//
// Hardware block scaling (`MX_ = true`): when the scales are powers of two (8-bit exponents,
// "UE8M0", chosen at quantisation) the tensor core applies them itself
// (`tcgen05.mma.kind::mxf8f6f4.block_scale`), reading one scale byte per operand row and 32
// K-elements from tensor memory, and the whole K loop accumulates in TMEM as in the unscaled
// kernels.  Four scale warps (one per TMEM lane quadrant) fetch the bytes of the next K blocks
// and store them into a ring of scale-factor columns beside the accumulators (tcgen05.st),
// one slot per ring stage; tiles are 128 x 192 so that two accumulators and the ring fit
// in the 512 columns.
//
// No load in this file is a cluster-multicast load.  Every wait is bounded: on a
// time-out the CTA raises its abort word (and its partner's), every role leaves
// its loop, in-flight copies get a grace period, TMEM is freed and the kernel
// returns with the status word set.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>

#include "../prim/cluster.cuh"
#include "../prim/tcgen05.cuh"
#include "../prim/tma.cuh"

namespace cb {

template <int BN_, int STAGES_, bool FP8_, int PAIR_ = 1, bool BS_ = false, bool MX_ = false>
struct GemmCfg {
  static constexpr bool MX = MX_;             // power-of-two block scales applied by the tensor core
  static constexpr int SF_BASE = 2 * BN_;     // first scale-factor column in TMEM (MX)
  static constexpr int SF_STRIDE = 16;        // columns per K block: 4 for A rows, up to 8 for B rows
  static constexpr int SF_SLOTS = 8;          // K blocks of scale factors in TMEM: 2 groups of 4
  static constexpr int PAIR = PAIR_;          // CTAs that share a tile (1, or 2 = a cluster)
  static constexpr bool BS = BS_;             // block-scaled fp8 with promotion in registers
  static constexpr int EPI_WARPS = BS_ ? 8 : 4;
  static constexpr int CTA_M = 128;           // accumulator rows per CTA
  static constexpr int BM = CTA_M * PAIR_;    // tile height
  static constexpr int BN = BN_;
  static constexpr int B_ROWS = BN_ / PAIR_;  // B rows each CTA loads
  static constexpr bool FP8 = FP8_;
  static constexpr int BK = FP8_ ? 128 : 64;  // elements per 128-byte row
  static constexpr int MMAS_PER_STAGE = 4;    // 128 B / 32 B per instruction
  static constexpr int STAGES = STAGES_;
  static constexpr int A_BYTES = CTA_M * 128;
  static constexpr int B_BYTES = B_ROWS * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_COLS = 64;                 // bf16 columns per store box (128 B)
  static constexpr int EPI_BUF_BYTES = 32 * 128;      // 32 rows x 128 B per warp and buffer
  static constexpr int EPI_BYTES = EPI_WARPS * 2 * EPI_BUF_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024;
  static constexpr int TMEM_COLS = MX_ ? 512 : 2 * BN;
  // Warp roles.  Plain: producer, MMA, 4 epilogue warps, signal warp.  Block-scaled: a
  // utility warp-group (producer, MMA, signal, one idle warp) that gives registers away and
  // two epilogue warp-groups that take them (setmaxnreg works on whole warp-groups).
  static constexpr int EPI_WARP0 = BS_ ? 4 : 2;
  static constexpr int SIGNAL_WARP = BS_ ? 2 : 6;
  static constexpr int SCALE_WARP0 = 8;       // MX: warps 8..11 write scale factors
  static constexpr int THREADS = (BS_ || MX_) ? 384 : 224;
  static_assert(!MX_ || (FP8_ && !BS_ && BN_ <= 192 &&
                         2 * BN_ + SF_SLOTS * SF_STRIDE <= 512),
                "hardware block scales: fp8, accumulators + scale ring within 512 TMEM columns");
  static_assert(!BS_ || (FP8_ && BN_ == 256), "block scales: fp8 operands, 256-column tiles");
  static_assert(PAIR_ == 1 || PAIR_ == 2, "one CTA or a pair per tile");
  static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "BN in {64,128,192,256}");
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS >= 32 && TMEM_COLS <= 512,
                "TMEM columns must be a power of two");
  static_assert(SMEM_BYTES <= 232448, "over the 227 KB shared-memory limit");
};

struct GemmShape {
  int M, N, K;
  int num_m_blocks, num_n_blocks, num_k_blocks;
  float alpha;
  // Block-scaled fp8 only: A scales [M, ceil(K/128)] and B scales [ceil(N/128), ceil(K/128)],
  // fp32, row-major (policies that gather A may supply their own through `a_scales`).
  const float* a_scale = nullptr;
  const float* b_scale = nullptr;
  // Hardware block scales only: exponent bytes, one per operand row and 128-wide K block,
  // packed four K blocks to a 32-bit word and stored K-group-major, word [kg * rows + row]
  // (B: one row per output column), so that the 32 lanes of a scale warp read 32 consecutive
  // words.  `sfa_rows` / `sfb_rows` are the row counts (pitches) of the two arrays.
  const uint32_t* sfa = nullptr;
  const uint32_t* sfb = nullptr;
  int sfa_rows = 0, sfb_rows = 0;
  // Optional role trace, 8 words per CTA of the launch (null = off): SM clock cycles the
  // MMA thread spent waiting for operands [0] and for a free accumulator [1] and its total
  // [2]; the producer's wait for free ring slots [3] and total [4]; the first epilogue
  // warp's wait for finished accumulators [5] and total [6].
  unsigned long long* trace = nullptr;
};

// Warp-collective mbar_wait: every lane of a converged warp calls it and all of them get the
// same answer (a lane that saw the barrier flip at the last moment must not go on alone to a
// `.sync.aligned` instruction or an election while its neighbours give up).  With tracing on,
// the waiting time is added to `*acc_cycles`.
__device__ __forceinline__ bool mbar_wait_traced(uint64_t* bar, uint32_t parity,
                                                 volatile int* abort_flag, uint32_t* status,
                                                 uint32_t detail, bool tracing,
                                                 long long* acc_cycles) {
  bool ok;
  if (!tracing) {
    ok = mbar_wait(bar, parity, abort_flag, status, detail);
  } else {
    // The whole call is timed: a try_wait may itself block for a while before it answers.
    const long long t0 = clock64();
    ok = mbar_wait(bar, parity, abort_flag, status, detail);
    *acc_cycles += clock64() - t0;
  }
  return __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
}

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
  uint64_t sf_full[2];    // scale warps -> MMA thread: a group of 4 K blocks of scale factors is in TMEM
  uint64_t sf_empty[2];   // MMA thread -> scale warps: the group's MMAs are done
  uint64_t sig_full[8];   // epilogue warps -> signal warp: a tile's stores were issued
  uint64_t sig_empty[8];  // signal warp -> epilogue warps: slot may be reused
  uint32_t tmem_base;
  int abort_flag;
  int a_ready_tiles;  // tiles whose A rows the producer has found ready (read by the scale warps)
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
//                                              were issued (one lane); quadrant = 4 * (CTA of
//                                              the pair) + epilogue warp, or 4 * CTA from the
//                                              signal warp of a direct policy
// Producer and MMA roles are executed by a whole, converged warp: every lane follows the loop
// and the waits, one elected lane issues the TMA loads / MMAs / commits.  Measured on B200
// with back-to-back MMAs of 32 pipe cycles each: 43-49 cycles per instruction issued this way
// against 61 (one CTA) / 82 (pair) from inside an `if (lane == 0)` branch, where the operands
// of every asynchronous instruction have to be moved out of a diverged thread's registers.
// At 4 MMAs + commits per 512 pipe cycles the branch form kept the tensor pipe idle a fifth
// of the time although the MMA thread never waited on a barrier.
template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_producer(const P& p, const GemmShape& g, uint8_t* ring,
                                              GemmCtl<Cfg::STAGES>* ctl, uint32_t* status,
                                              int cta, int num_ctas, int sub) {
  uint32_t stage = 0, phase = 0;
  const int ntiles = Policy::num_tiles(p);
  const bool tracing = g.trace != nullptr;
  long long w_empty = 0;
  const long long t_begin = tracing ? clock64() : 0;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t ring_addr = smem_u32(ring);
  const uint32_t full0 = smem_u32(&ctl->full[0]);
  int ready_tiles = 0;
  // Pair: both CTAs' bytes are counted on the even CTA's barrier, the one its MMA warp waits on.
  const uint32_t full0_leader = Cfg::PAIR == 2 ? map_to_cta(full0, 0) : full0;
  for (int tile = cta; tile < ntiles; tile += num_ctas) {
    int m_blk, n_blk;
    Policy::tile_coord(p, tile, &m_blk, &n_blk);
    // The readiness wait polls a word that peers write: one lane only.
    int ready = 1;
    if (lane == 0) ready = Policy::wait_a_ready(p, m_blk, &ctl->abort_flag) ? 1 : 0;
    if (__shfl_sync(0xffffffffu, ready, 0) == 0) return;
    if constexpr (Cfg::MX) {
      if (lane == 0) {
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&ctl->a_ready_tiles) = ++ready_tiles;
      }
    }
    const CUtensorMap* ma = Policy::map_a(p, m_blk);
    const CUtensorMap* mb = Policy::map_b(p);
    const int arow = Policy::a_row(p, m_blk) + sub * Cfg::CTA_M;
    const int brow = Policy::b_row(p, m_blk, n_blk) + sub * Cfg::B_ROWS;
    for (int kb = 0; kb < g.num_k_blocks; ++kb) {
      if (!mbar_wait_traced(&ctl->empty[stage], phase ^ 1u, &ctl->abort_flag, status,
                            0x100 + stage, tracing, &w_empty))
        return;
      if (elect_one()) {
        const uint32_t sa = ring_addr + stage * Cfg::STAGE_BYTES;
        const uint32_t sb = sa + Cfg::A_BYTES;
        if constexpr (Cfg::PAIR == 2) {
          // The partner's bytes may land before this expect_tx: the transaction count is
          // allowed to run negative within a phase.
          if (sub == 0) mbar_arrive_expect_tx_addr(full0 + stage * 8u, 2 * Cfg::STAGE_BYTES);
          const uint32_t bar = full0_leader + stage * 8u;
          tma_load_2d_pair(sa, ma, kb * Cfg::BK, arow, bar);
          tma_load_2d_pair(sb, mb, kb * Cfg::BK, brow, bar);
        } else {
          const uint32_t bar = full0 + stage * 8u;
          mbar_arrive_expect_tx_addr(bar, Cfg::STAGE_BYTES);
          tma_load_2d_addr(sa, ma, kb * Cfg::BK, arow, bar);
          tma_load_2d_addr(sb, mb, kb * Cfg::BK, brow, bar);
        }
      }
      __syncwarp();
      if (++stage == Cfg::STAGES) {
        stage = 0;
        phase ^= 1u;
      }
    }
  }
  if (tracing && lane == 0) {
    g.trace[blockIdx.x * 8 + 3] = static_cast<unsigned long long>(w_empty);
    g.trace[blockIdx.x * 8 + 4] = static_cast<unsigned long long>(clock64() - t_begin);
  }
}

template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_mma(const P& p, const GemmShape& g, uint8_t* ring,
                                         GemmCtl<Cfg::STAGES>* ctl, uint32_t* status, int cta,
                                         int num_ctas, uint32_t tmem_base) {
  constexpr uint32_t idesc = make_idesc(Cfg::BM, Cfg::BN, Cfg::FP8 ? 0u : 1u);  // M = 256 for a pair
  uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
  const int ntiles = Policy::num_tiles(p);
  const bool tracing = g.trace != nullptr;
  long long w_full = 0, w_acc = 0;
  const long long t_begin = tracing ? clock64() : 0;
  const uint32_t lane = threadIdx.x & 31u;
  // Descriptors and barrier addresses of stage 0; a stage further is a constant step.
  const uint64_t a_desc0 = make_sw128_kmajor_desc(smem_u32(ring));
  constexpr uint64_t kStageStep = static_cast<uint64_t>(Cfg::STAGE_BYTES >> 4);
  constexpr uint64_t kBStep = static_cast<uint64_t>(Cfg::A_BYTES >> 4);
  const uint32_t empty0 = smem_u32(&ctl->empty[0]);
  const uint32_t tfull0 = smem_u32(&ctl->tmem_full[0]);
  const uint32_t empty0_peer = Cfg::PAIR == 2 ? map_to_cta(empty0, 1) : 0u;
  const uint32_t tfull0_peer = Cfg::PAIR == 2 ? map_to_cta(tfull0, 1) : 0u;
  for (int tile = cta; tile < ntiles; tile += num_ctas) {
    if (!mbar_wait_traced(&ctl->tmem_empty[acc], acc_phase ^ 1u, &ctl->abort_flag, status,
                          0x200 + acc, tracing, &w_acc))
      return;
    tc_fence_after_sync();
    const uint32_t d_tmem = tmem_base + acc * Cfg::BN;
    for (int kb = 0; kb < g.num_k_blocks; ++kb) {
      if (!mbar_wait_traced(&ctl->full[stage], phase, &ctl->abort_flag, status, 0x300 + stage,
                            tracing, &w_full))
        return;
      tc_fence_after_sync();
      // operands computed warp-uniformly, outside the elected region
      const uint64_t a_desc = a_desc0 + stage * kStageStep;
      const uint64_t b_desc = a_desc + kBStep;
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < Cfg::MMAS_PER_STAGE; ++k) {
          // 32 bytes along K per instruction: +2 in the descriptor's 16-byte address units.
          const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
          if constexpr (Cfg::PAIR == 2) {
            if constexpr (Cfg::FP8)
              mma_fp8_ss_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, accum);
            else
              mma_bf16_ss_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, accum);
          } else {
            if constexpr (Cfg::FP8)
              mma_fp8_ss(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, accum);
            else
              mma_bf16_ss(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, accum);
          }
        }
        // The ring slot is free once these MMAs have read it (in both CTAs of a pair).
        if constexpr (Cfg::PAIR == 2) {
          mma_commit_pair(empty0 + stage * 8u);
          mma_commit_pair(empty0_peer + stage * 8u);
        } else {
          mma_commit_addr(empty0 + stage * 8u);
        }
      }
      __syncwarp();
      if (++stage == Cfg::STAGES) {
        stage = 0;
        phase ^= 1u;
      }
    }
    // Accumulator complete.
    if (elect_one()) {
      if constexpr (Cfg::PAIR == 2) {
        mma_commit_pair(tfull0 + acc * 8u);
        mma_commit_pair(tfull0_peer + acc * 8u);
      } else {
        mma_commit_addr(tfull0 + acc * 8u);
      }
    }
    __syncwarp();
    acc ^= 1u;
    if (acc == 0u) acc_phase ^= 1u;
  }
  if (tracing && lane == 0) {
    g.trace[blockIdx.x * 8 + 0] = static_cast<unsigned long long>(w_full);
    g.trace[blockIdx.x * 8 + 1] = static_cast<unsigned long long>(w_acc);
    g.trace[blockIdx.x * 8 + 2] = static_cast<unsigned long long>(clock64() - t_begin);
  }
}

// MMA role with block scales: every 128-wide K block gets a fresh accumulator, the two TMEM
// buffers alternating; `tmem_full[b]` / `tmem_empty[b]` are handed over once per K block.
template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_mma_bs(const P& p, const GemmShape& g, uint8_t* ring,
                                            GemmCtl<Cfg::STAGES>* ctl, uint32_t* status, int cta,
                                            int num_ctas, uint32_t tmem_base) {
  constexpr uint32_t idesc = make_idesc(Cfg::BM, Cfg::BN, 0u);
  uint32_t stage = 0, phase = 0, buf = 0, buf_phase = 0;
  const int ntiles = Policy::num_tiles(p);
  const uint64_t a_desc0 = make_sw128_kmajor_desc(smem_u32(ring));
  constexpr uint64_t kStageStep = static_cast<uint64_t>(Cfg::STAGE_BYTES >> 4);
  constexpr uint64_t kBStep = static_cast<uint64_t>(Cfg::A_BYTES >> 4);
  const uint32_t empty0 = smem_u32(&ctl->empty[0]);
  const uint32_t tfull0 = smem_u32(&ctl->tmem_full[0]);
  const uint32_t empty0_peer = Cfg::PAIR == 2 ? map_to_cta(empty0, 1) : 0u;
  const uint32_t tfull0_peer = Cfg::PAIR == 2 ? map_to_cta(tfull0, 1) : 0u;
  for (int tile = cta; tile < ntiles; tile += num_ctas) {
    for (int kb = 0; kb < g.num_k_blocks; ++kb) {
      if (!mbar_wait_traced(&ctl->tmem_empty[buf], buf_phase ^ 1u, &ctl->abort_flag, status,
                            0x200 + buf, false, nullptr))
        return;
      if (!mbar_wait_traced(&ctl->full[stage], phase, &ctl->abort_flag, status, 0x300 + stage,
                            false, nullptr))
        return;
      tc_fence_after_sync();
      if (elect_one()) {
        const uint32_t d_tmem = tmem_base + buf * Cfg::BN;
        const uint64_t a_desc = a_desc0 + stage * kStageStep;
        const uint64_t b_desc = a_desc + kBStep;
#pragma unroll
        for (int k = 0; k < Cfg::MMAS_PER_STAGE; ++k) {
          if constexpr (Cfg::PAIR == 2)
            mma_fp8_ss_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, k > 0 ? 1u : 0u);
          else
            mma_fp8_ss(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, k > 0 ? 1u : 0u);
        }
        if constexpr (Cfg::PAIR == 2) {
          mma_commit_pair(empty0 + stage * 8u);
          mma_commit_pair(empty0_peer + stage * 8u);
          mma_commit_pair(tfull0 + buf * 8u);
          mma_commit_pair(tfull0_peer + buf * 8u);
        } else {
          mma_commit_addr(empty0 + stage * 8u);
          mma_commit_addr(tfull0 + buf * 8u);
        }
      }
      __syncwarp();
      if (++stage == Cfg::STAGES) {
        stage = 0;
        phase ^= 1u;
      }
      buf ^= 1u;
      if (buf == 0u) buf_phase ^= 1u;
    }
  }
}

// MMA role with hardware block scales: as gemm_mma, plus the wait for the stage's scale
// factors and the scale-factor operands of the instruction.
template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_mma_mx(const P& p, const GemmShape& g, uint8_t* ring,
                                            GemmCtl<Cfg::STAGES>* ctl, uint32_t* status, int cta,
                                            int num_ctas, uint32_t tmem_base) {
  uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
  const int ntiles = Policy::num_tiles(p);
  const uint64_t a_desc0 = make_sw128_kmajor_desc(smem_u32(ring));
  constexpr uint64_t kStageStep = static_cast<uint64_t>(Cfg::STAGE_BYTES >> 4);
  constexpr uint64_t kBStep = static_cast<uint64_t>(Cfg::A_BYTES >> 4);
  const uint32_t empty0 = smem_u32(&ctl->empty[0]);
  const uint32_t tfull0 = smem_u32(&ctl->tmem_full[0]);
  const uint32_t sfe0 = smem_u32(&ctl->sf_empty[0]);
  const uint32_t empty0_peer = Cfg::PAIR == 2 ? map_to_cta(empty0, 1) : 0u;
  const uint32_t tfull0_peer = Cfg::PAIR == 2 ? map_to_cta(tfull0, 1) : 0u;
  const uint32_t sfe0_peer = Cfg::PAIR == 2 ? map_to_cta(sfe0, 1) : 0u;
  uint32_t gcount = 0;  // groups of 4 K blocks so far (a tile starts a new group)
  const bool tracing = g.trace != nullptr;  // [0] operands, [1] accumulator + scale factors
  long long w_full = 0, w_other = 0;
  const long long t_begin = tracing ? clock64() : 0;
  for (int tile = cta; tile < ntiles; tile += num_ctas) {
    if (!mbar_wait_traced(&ctl->tmem_empty[acc], acc_phase ^ 1u, &ctl->abort_flag, status,
                          0x200 + acc, tracing, &w_other))
      return;
    tc_fence_after_sync();
    const uint32_t d_tmem = tmem_base + acc * Cfg::BN;
    for (int kb = 0; kb < g.num_k_blocks; ++kb) {
      const uint32_t grp = gcount & 1u;
      if ((kb & 3) == 0 &&
          !mbar_wait_traced(&ctl->sf_full[grp], (gcount >> 1) & 1u, &ctl->abort_flag, status,
                            0x380 + grp, tracing, &w_other))
        return;
      if (!mbar_wait_traced(&ctl->full[stage], phase, &ctl->abort_flag, status, 0x300 + stage,
                            tracing, &w_full))
        return;
      tc_fence_after_sync();
      const bool group_ends = (kb & 3) == 3 || kb == g.num_k_blocks - 1;
      // Operands are computed by the whole (converged) warp, so they can live in uniform
      // registers; only the asynchronous instructions themselves sit under the election.
      const uint64_t a_desc = a_desc0 + stage * kStageStep;
      const uint64_t b_desc = a_desc + kBStep;
      const uint32_t sfa =
          tmem_base + Cfg::SF_BASE + (grp * 4u + static_cast<uint32_t>(kb & 3)) * Cfg::SF_STRIDE;
      const uint32_t sfb = sfa + 4u;
      const uint32_t first = kb > 0 ? 1u : 0u;
      if (elect_one()) {
        // Four K steps of 32; step j takes byte j of the scale columns.
        if constexpr (Cfg::PAIR == 2) {
          mma_mxf8_ss_pair(d_tmem, a_desc, b_desc, make_idesc_mx(Cfg::BM, Cfg::BN, 0u), sfa, sfb, first);
          mma_mxf8_ss_pair(d_tmem, a_desc + 2u, b_desc + 2u, make_idesc_mx(Cfg::BM, Cfg::BN, 1u), sfa, sfb, 1u);
          mma_mxf8_ss_pair(d_tmem, a_desc + 4u, b_desc + 4u, make_idesc_mx(Cfg::BM, Cfg::BN, 2u), sfa, sfb, 1u);
          mma_mxf8_ss_pair(d_tmem, a_desc + 6u, b_desc + 6u, make_idesc_mx(Cfg::BM, Cfg::BN, 3u), sfa, sfb, 1u);
          mma_commit_pair(empty0 + stage * 8u);
          mma_commit_pair(empty0_peer + stage * 8u);
          if (group_ends) {  // the group's scale columns are free, in both CTAs
            mma_commit_pair(sfe0 + grp * 8u);
            mma_commit_pair(sfe0_peer + grp * 8u);
          }
        } else {
          mma_mxf8_ss(d_tmem, a_desc, b_desc, make_idesc_mx(Cfg::BM, Cfg::BN, 0u), sfa, sfb, first);
          mma_mxf8_ss(d_tmem, a_desc + 2u, b_desc + 2u, make_idesc_mx(Cfg::BM, Cfg::BN, 1u), sfa, sfb, 1u);
          mma_mxf8_ss(d_tmem, a_desc + 4u, b_desc + 4u, make_idesc_mx(Cfg::BM, Cfg::BN, 2u), sfa, sfb, 1u);
          mma_mxf8_ss(d_tmem, a_desc + 6u, b_desc + 6u, make_idesc_mx(Cfg::BM, Cfg::BN, 3u), sfa, sfb, 1u);
          mma_commit_addr(empty0 + stage * 8u);
          if (group_ends) mma_commit_addr(sfe0 + grp * 8u);  // the group's scale columns are free
        }
      }
      __syncwarp();
      if (group_ends) ++gcount;
      if (++stage == Cfg::STAGES) {
        stage = 0;
        phase ^= 1u;
      }
    }
    if (elect_one()) {
      if constexpr (Cfg::PAIR == 2) {
        mma_commit_pair(tfull0 + acc * 8u);
        mma_commit_pair(tfull0_peer + acc * 8u);
      } else {
        mma_commit_addr(tfull0 + acc * 8u);
      }
    }
    __syncwarp();
    acc ^= 1u;
    if (acc == 0u) acc_phase ^= 1u;
  }
  if (tracing && (threadIdx.x & 31u) == 0) {
    g.trace[blockIdx.x * 8 + 0] = static_cast<unsigned long long>(w_full);
    g.trace[blockIdx.x * 8 + 1] = static_cast<unsigned long long>(w_other);
    g.trace[blockIdx.x * 8 + 2] = static_cast<unsigned long long>(clock64() - t_begin);
  }
}

// Packed exponent words of the A rows of a tile (K group 0; a K group further is `*pitch`
// words on): GemmShape::sfa at the policy's A row, unless the policy gathered A from other ranks
// and names its own source (`a_sf(p, m_blk, &pitch)`).
template <class Policy, class P>
__device__ __forceinline__ const uint32_t* tile_a_sf(const P& p, const GemmShape& g, int m_blk,
                                                     long long* pitch) {
  if constexpr (requires { Policy::a_sf(p, m_blk, pitch); }) {
    return Policy::a_sf(p, m_blk, pitch);
  } else {
    *pitch = g.sfa_rows;
    return g.sfa + Policy::a_row(p, m_blk);
  }
}

// Scale warp (one per TMEM lane quadrant; all four write the same data, the layout wants it
// replicated): lane l holds rows l, l+32, l+64, l+96 of A and l, l+32, ... of the B tile.  It
// works in groups of four K blocks - one 32-bit load per row brings their four exponent bytes,
// the next group's loads in flight meanwhile - and two groups of TMEM columns alternate: wait
// until the MMAs of the group's previous use are done, store 4 x (4 + 8) columns, one
// tcgen05.wait::st, one arrival.
template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_scale_writer(const P& p, const GemmShape& g,
                                                  GemmCtl<Cfg::STAGES>* ctl, uint32_t* status,
                                                  int cta, int num_ctas, uint32_t tmem_base,
                                                  uint32_t warp, uint32_t lane, int sub) {
  constexpr int NB = Cfg::BN / 32;  // B-row groups of this tile (<= 8)
  const uint32_t q = warp & 3u;
  uint32_t gcount = 0;  // groups of 4 K blocks so far, in step with the MMA role
  int tcount = 0;       // tiles so far, against the producer's count of tiles whose A rows are there
  const int ntiles = Policy::num_tiles(p);
  const int nkb = g.num_k_blocks;
  const uint32_t t0 = tmem_base + ((q * 32u) << 16) + Cfg::SF_BASE;
  constexpr uint32_t kOne = 0x7f7f7f7fu;  // exponent 127 = 1.0, for rows outside the operands
  for (int tile = cta; tile < ntiles; tile += num_ctas) {
    int m_blk, n_blk;
    Policy::tile_coord(p, tile, &m_blk, &n_blk);
    // this CTA's 128 rows of the tile; all BN columns of B
    // A tile whose A rows come from another rank: its scale words arrive with the rows.  The
    // producer waits for them before its first load of the tile and then counts the tile in
    // `a_ready_tiles`; this warp follows that count.
    {
      int ok = 1;
      if (lane == 0) {
        uint64_t t_start = 0;
        for (uint32_t it = 0; *reinterpret_cast<volatile int*>(&ctl->a_ready_tiles) <= tcount; ++it) {
          if ((it & 63u) == 63u) {
            if (*reinterpret_cast<volatile int*>(&ctl->abort_flag) != 0) { ok = 0; break; }
            const uint64_t now = globaltimer_ns();
            if (t_start == 0) t_start = now;
            if (now - t_start > CB_MBAR_TIMEOUT_NS) {
              ctl->abort_flag = 1;
              report_status(status, CB_TIMEOUT_MBARRIER, 0, 0x580);
              ok = 0;
              break;
            }
          }
        }
        __threadfence_block();
      }
      if (__shfl_sync(0xffffffffu, ok, 0) == 0) return;
      ++tcount;
    }
    long long pitch_a = 0;
    const uint32_t* pa = tile_a_sf<Policy>(p, g, m_blk, &pitch_a) + sub * Cfg::CTA_M;
    const int a_rows_left = g.M - m_blk * Cfg::BM - sub * Cfg::CTA_M;
    const int b_row0 = Policy::b_row(p, m_blk, n_blk);
    const int b_rows_left = g.N - n_blk * Cfg::BN;
    auto load_group = [&](int kb, uint32_t (&wa)[4], uint32_t (&wb)[NB]) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int r = c * 32 + static_cast<int>(lane);
        // L2-coherent load: the words of gathered rows were written by a peer during this launch
        wa[c] = (kb < nkb && r < a_rows_left) ? __ldcg(pa + (kb >> 2) * pitch_a + r) : kOne;
      }
#pragma unroll
      for (int c = 0; c < NB; ++c) {
        const int r = c * 32 + static_cast<int>(lane);
        wb[c] = (kb < nkb && r < b_rows_left)
                    ? __ldg(g.sfb + static_cast<long long>(kb >> 2) * g.sfb_rows + b_row0 + r)
                    : kOne;
      }
    };
    uint32_t wa[4], wb[NB], na[4], nb[NB];
    load_group(0, wa, wb);
    for (int kg = 0; kg < nkb; kg += 4) {
      load_group(kg + 4, na, nb);  // in flight while this group is written
      const uint32_t grp = gcount & 1u;
      if (!mbar_wait_traced(&ctl->sf_empty[grp], ((gcount >> 1) & 1u) ^ 1u, &ctl->abort_flag,
                            status, 0x500 + grp, false, nullptr))
        return;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t ra[4], rb[8];
#pragma unroll
        for (int c = 0; c < 4; ++c) ra[c] = ((wa[c] >> (8 * j)) & 0xffu) * 0x01010101u;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          rb[c] = c < NB ? ((wb[c < NB ? c : 0] >> (8 * j)) & 0xffu) * 0x01010101u : kOne;
        const uint32_t t = t0 + (grp * 4u + j) * Cfg::SF_STRIDE;
        tmem_st_32x4(t, ra);
        tmem_st_32x8(t + 4u, rb);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (Cfg::PAIR == 2 && sub != 0)
          mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->sf_full[grp]), 0));
        else
          mbar_arrive(&ctl->sf_full[grp]);
      }
      ++gcount;
#pragma unroll
      for (int c = 0; c < 4; ++c) wa[c] = na[c];
#pragma unroll
      for (int c = 0; c < NB; ++c) wb[c] = nb[c];
    }
  }
}

// One epilogue warp has read accumulator `acc` for the last time: tell the MMA thread (which
// lives in the even CTA of a pair).
template <class Cfg>
__device__ __forceinline__ void release_accumulator(GemmCtl<Cfg::STAGES>* ctl, uint32_t acc,
                                                    int sub) {
  if constexpr (Cfg::PAIR == 2) {
    if (sub != 0) {
      mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->tmem_empty[acc]), 0));
      return;
    }
  }
  mbar_arrive(&ctl->tmem_empty[acc]);
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

// A direct policy may declare `static constexpr bool kReduceLocal = true`: tiles for which
// `tile_is_local(p, m_blk)` holds are then not sent anywhere; the epilogue adds the staged
// partial tiles that other ranks sent for them (fp32, fixed order) to its own accumulator
// and writes the final rows, so the reduction of a reduce-scatter overlaps the main loop of
// the next tile and the local partial never travels through memory.
//   bool tile_is_local(const P&, int m_blk)
//   bool wait_local_ready(const P&, int m_blk, int n_blk, int sub)   (one lane per warp)
//   void local_reduce(const P&, int m_blk, int n_blk, LocalReduce*)
struct LocalReduce {
  int nsrc;               // staged copies to add (0..7)
  const uint8_t* src[7];  // address of (tile row 0, tile column 0) in each copy
  long long src_ld;       // row pitch of the copies, bytes
  uint8_t* out;           // address of (tile row 0, tile column 0) of the result
  long long out_ld;
};
template <class Policy>
__host__ __device__ constexpr bool policy_reduce_local() {
  if constexpr (requires { Policy::kReduceLocal; }) {
    return Policy::kReduceLocal;
  } else {
    return false;
  }
}

// bf16x8 (+)= bf16x8 in fp32.
__device__ __forceinline__ void acc_bf16x8(float (&a)[8], const uint4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 t = __bfloat1622float2(h[k]);
    a[2 * k] += t.x;
    a[2 * k + 1] += t.y;
  }
}

// Second half of the direct epilogue for one 128-column half `h` of the tile: the 32 x 256 B
// staging buffer `buf` of this warp holds the bf16 rows; a half-warp takes a row and either
// stores it to the policy's destinations or, for a tile that is reduced in place, adds the
// staged partial copies and stores the final row.
template <class Cfg, class Policy, class P>
__device__ __forceinline__ void direct_store_half(const P& p, uint8_t* buf, uint32_t lane,
                                                  uint32_t q, int h, int CH, int sub, int m_blk,
                                                  int n_blk, const DirectTargets& tg,
                                                  bool local_tile, const LocalReduce& lr) {
  constexpr bool kReduce = policy_reduce_local<Policy>();
  __syncwarp();
  // Half-warp per row: 16 lanes x 16 B = 256 B (128 bf16 columns; 64 when BN == 64).
  const uint32_t idx = lane & 15u;
  const int col = h * 128 + static_cast<int>(idx) * 8;
  const bool col_ok = (static_cast<int>(idx) < CH * 8) && col < tg.cols;
  if constexpr (kReduce) {
    if (local_tile) {
      // Two rows per lane and step, every staged copy of both loaded before the sums.
#pragma unroll 1
      for (int i0 = 0; i0 < 16; i0 += 2) {
        uint4 parts[2][7];
        bool okr[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t r = 2u * (i0 + u) + (lane >> 4);
          const int row = sub * Cfg::CTA_M + static_cast<int>(q * 32u + r);
          okr[u] = col_ok && row < tg.rows;
          const long long off = row * lr.src_ld + col * 2ll;
#pragma unroll
          for (int sidx = 0; sidx < 7; ++sidx)
            if (okr[u] && sidx < lr.nsrc)
              parts[u][sidx] = __ldcg(reinterpret_cast<const uint4*>(lr.src[sidx] + off));
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (!okr[u]) continue;
          const uint32_t r = 2u * (i0 + u) + (lane >> 4);
          const int row = sub * Cfg::CTA_M + static_cast<int>(q * 32u + r);
          const uint4 own =
              *reinterpret_cast<const uint4*>(buf + r * 256u + ((idx ^ (r & 7u)) * 16u));
          float a[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) a[k] = 0.f;
          acc_bf16x8(a, own);
#pragma unroll
          for (int sidx = 0; sidx < 7; ++sidx)
            if (sidx < lr.nsrc) acc_bf16x8(a, parts[u][sidx]);
          uint4 o;
          __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int k = 0; k < 4; ++k) oh[k] = __floats2bfloat162_rn(a[2 * k], a[2 * k + 1]);
          st_v4(lr.out + row * lr.out_ld + col * 2ll, o);
        }
      }
      __syncwarp();
      return;
    }
  }
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const uint32_t r = 2u * i + (lane >> 4);
    const int row = sub * Cfg::CTA_M + static_cast<int>(q * 32u + r);
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

// Epilogue for policies with `kDirect`: accumulator -> bf16 -> shared memory
// (transposition) -> row-contiguous 16-byte global stores, 256 bytes per row and
// half-warp.  Used where the destination is another GPU: load/store traffic
// keeps NVLink busy with few SMs, and no TMA store sits between data and flag.
template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_epilogue_direct(const P& p, const GemmShape& g,
                                                     uint8_t* epi_smem,
                                                     GemmCtl<Cfg::STAGES>* ctl, uint32_t* status,
                                                     int cta, int num_ctas, uint32_t tmem_base,
                                                     uint32_t warp, uint32_t lane, int sub) {
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
    if (!mbar_wait_traced(&ctl->tmem_full[acc], acc_phase, &ctl->abort_flag, status, 0x400 + acc,
                          false, nullptr))
      return;
    tc_fence_after_sync();
    constexpr bool kReduce = policy_reduce_local<Policy>();
    bool local_tile = false;
    LocalReduce lr;
    if constexpr (kReduce) {
      local_tile = Policy::tile_is_local(p, m_blk);
      if (local_tile) {
        Policy::local_reduce(p, m_blk, n_blk, &lr);
        int ok = 1;
        if (lane == 0 && lr.nsrc > 0) ok = Policy::wait_local_ready(p, m_blk, n_blk, sub) ? 1 : 0;
        if (__shfl_sync(0xffffffffu, ok, 0) == 0) {
          ctl->abort_flag = 1;
          return;
        }
      }
    }
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
          if (lane == 0) release_accumulator<Cfg>(ctl, acc, sub);
        }
        epi_write_row_256(buf, lane, cc, r0, r1, g.alpha);
      }
      direct_store_half<Cfg, Policy>(p, buf, lane, q, h, CH, sub, m_blk, n_blk, tg, local_tile, lr);
    }
    // Hand the tile to the signal warp: it runs the (slow, ~20 us under store traffic)
    // system-scope fence and raises the flag while these warps go on with the next tile.
    __syncwarp();
    if (Policy::kSignalPerTile && !local_tile) {
      if (lane == 0) {
        const uint32_t slot = seq & 7u;
        if (!mbar_wait(&ctl->sig_empty[slot], ((seq >> 3) & 1u) ^ 1u, &ctl->abort_flag, status,
                       0x800 + slot))
          return;
        mbar_arrive(&ctl->sig_full[slot]);
      }
      ++seq;  // sequence of signalled tiles only
    }
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
                                            uint32_t* status, int cta, int num_ctas, int sub) {
  uint32_t seq = 0;
  const int ntiles = Policy::num_tiles(p);
  int pend_m[4], pend_n[4];
  int npend = 0;
  int tile = cta;
  while (tile < ntiles || npend > 0) {
    if constexpr (policy_reduce_local<Policy>()) {
      // Tiles that are reduced in place are not signalled to anybody.
      if (tile < ntiles) {
        int m_blk, n_blk;
        Policy::tile_coord(p, tile, &m_blk, &n_blk);
        if (Policy::tile_is_local(p, m_blk)) {
          tile += num_ctas;
          continue;
        }
      }
    }
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
    for (int i = 0; i < npend; ++i) Policy::tile_done(p, pend_m[i], pend_n[i], sub * 4);
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
                                                  uint32_t lane, int sub) {
  const uint32_t q = warp & 3u;  // TMEM lane quadrant this warp may read
  uint8_t* bufs = epi_smem + q * (2 * Cfg::EPI_BUF_BYTES);
  uint32_t acc = 0, acc_phase = 0, buf = 0;
  const int ntiles = Policy::num_tiles(p);
  const bool tracing = g.trace != nullptr && q == 0 && lane == 0;
  long long w_tfull = 0;
  const long long t_begin = tracing ? clock64() : 0;
  for (int tile = cta; tile < ntiles; tile += num_ctas) {
    int m_blk, n_blk;
    Policy::tile_coord(p, tile, &m_blk, &n_blk);
    if (!mbar_wait_traced(&ctl->tmem_full[acc], acc_phase, &ctl->abort_flag, status, 0x400 + acc,
                          tracing, &w_tfull))
      return;
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
        if (lane == 0) release_accumulator<Cfg>(ctl, acc, sub);
      }
      // The buffer we are about to fill was read by the store issued two boxes ago.
      if (lane == 0) bulk_wait_read<1>();
      __syncwarp();
      uint8_t* b = bufs + buf * Cfg::EPI_BUF_BYTES;
      epi_write_row_swizzled(b, lane, r0, r1, kGated ? 1.0f : g.alpha);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        Policy::store_box(p, m_blk, n_blk, sub * Cfg::CTA_M + static_cast<int>(q * 32u),
                          c * Cfg::EPI_COLS, b);
        bulk_commit();
      }
      buf ^= 1u;
    }
    if (lane == 0) Policy::tile_done(p, m_blk, n_blk, sub * 4 + static_cast<int>(q));
    acc ^= 1u;
    if (acc == 0u) acc_phase ^= 1u;
  }
  if (lane == 0) bulk_wait_all<0>();
  if (tracing) {
    g.trace[blockIdx.x * 8 + 5] = static_cast<unsigned long long>(w_tfull);
    g.trace[blockIdx.x * 8 + 6] = static_cast<unsigned long long>(clock64() - t_begin);
  }
}

__device__ __forceinline__ uint64_t pack_u32x2(uint32_t lo, uint32_t hi) {
  return static_cast<uint64_t>(lo) | (static_cast<uint64_t>(hi) << 32);
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  return pack_u32x2(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
template <int N>
__device__ __forceinline__ void warpgroup_reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void warpgroup_reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// Where the scales of a tile come from: by default the arrays of GemmShape, indexed by the
// policy's A / B row coordinates; a policy whose A rows were gathered from other ranks names
// its own source with `static const float* a_scales(const P&, int m_blk)` (scales of the
// tile's first row, K-block-major per row).
template <class Policy, class P, class Cfg>
__device__ __forceinline__ const float* tile_a_scales(const P& p, const GemmShape& g, int m_blk) {
  if constexpr (requires { Policy::a_scales(p, m_blk); }) {
    return Policy::a_scales(p, m_blk);
  } else {
    return g.a_scale + static_cast<long long>(Policy::a_row(p, m_blk)) * g.num_k_blocks;
  }
}

// Epilogue warps of the block-scaled kernel: promotion of every K block's partial sum into
// registers, then the usual conversion and store (TMA boxes, or the direct / reducing path).
// Epilogue warp e of the eight reads TMEM lane quadrant (warp index) % 4 (a hardware rule)
// and the 128-column half h = e / 4 of the tile, which is exactly one 128 x 128 block of B.
// The running sums are kept as packed pairs and updated with two-wide FMAs.
template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_epilogue_bs(const P& p, const GemmShape& g, uint8_t* epi_smem,
                                                 GemmCtl<Cfg::STAGES>* ctl, uint32_t* status,
                                                 int cta, int num_ctas, uint32_t tmem_base,
                                                 uint32_t warp, uint32_t lane, int sub) {
  const uint32_t q = warp & 3u;
  const uint32_t ew = warp - Cfg::EPI_WARP0;  // 0..7
  const int h = static_cast<int>(ew >> 2);
  uint8_t* bufs = epi_smem + ew * (2 * Cfg::EPI_BUF_BYTES);
  uint32_t buf = 0, buf_phase = 0, seq = 0, sbuf = 0;
  const int ntiles = Policy::num_tiles(p);
  const int nkb = g.num_k_blocks;
  for (int tile = cta; tile < ntiles; tile += num_ctas) {
    int m_blk, n_blk;
    Policy::tile_coord(p, tile, &m_blk, &n_blk);
    const int row_in_tile = sub * Cfg::CTA_M + static_cast<int>(q * 32u + lane);
    // scales of this thread's row and of this warp's block of B
    const float* as = tile_a_scales<Policy, P, Cfg>(p, g, m_blk) +
                      static_cast<long long>(row_in_tile) * nkb;
    const bool row_ok = m_blk * Cfg::BM + row_in_tile < g.M;  // rows past M read no scale
    const int b_blk = (Policy::b_row(p, m_blk, n_blk) >> 7) + h;
    const bool bcol_ok = n_blk * Cfg::BN + h * 128 < g.N;
    const float* bs = g.b_scale + static_cast<long long>(b_blk) * nkb;
    uint64_t acc2[64];  // 128 fp32 sums as pairs
#pragma unroll
    for (int i = 0; i < 64; ++i) acc2[i] = 0ull;
    for (int kb = 0; kb < nkb; ++kb) {
      const float f = (row_ok && bcol_ok) ? __ldg(as + kb) * __ldg(bs + kb) : 0.f;
      const uint64_t f2 = pack_f32x2(f, f);
      if (!mbar_wait_traced(&ctl->tmem_full[buf], buf_phase, &ctl->abort_flag, status,
                            0x400 + buf, false, nullptr))
        return;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((q * 32u) << 16) + buf * Cfg::BN + h * 128;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(taddr + c * 64, r0);
        tmem_ld_32x32(taddr + c * 64 + 32, r1);
        tmem_wait_ld();
        if (c == 1) {
          // last read of this partial sum: the MMA thread may start the K block after next
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) release_accumulator<Cfg>(ctl, buf, sub);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          acc2[c * 32 + i] = fma_f32x2(pack_u32x2(r0[2 * i], r0[2 * i + 1]), f2, acc2[c * 32 + i]);
          acc2[c * 32 + 16 + i] =
              fma_f32x2(pack_u32x2(r1[2 * i], r1[2 * i + 1]), f2, acc2[c * 32 + 16 + i]);
        }
      }
      buf ^= 1u;
      if (buf == 0u) buf_phase ^= 1u;
    }
    // ---- store: two 64-column chunks of this warp's half
    if constexpr (Policy::kDirect) {
      DirectTargets tg;
      Policy::direct_targets(p, m_blk, n_blk, &tg);
      constexpr bool kReduce = policy_reduce_local<Policy>();
      bool local_tile = false;
      LocalReduce lr;
      if constexpr (kReduce) {
        local_tile = Policy::tile_is_local(p, m_blk);
        if (local_tile) {
          Policy::local_reduce(p, m_blk, n_blk, &lr);
          int ok = 1;
          if (lane == 0 && lr.nsrc > 0) ok = Policy::wait_local_ready(p, m_blk, n_blk, sub) ? 1 : 0;
          if (__shfl_sync(0xffffffffu, ok, 0) == 0) {
            ctl->abort_flag = 1;
            return;
          }
        }
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r0[32], r1[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          r0[2 * i] = static_cast<uint32_t>(acc2[c * 32 + i]);
          r0[2 * i + 1] = static_cast<uint32_t>(acc2[c * 32 + i] >> 32);
          r1[2 * i] = static_cast<uint32_t>(acc2[c * 32 + 16 + i]);
          r1[2 * i + 1] = static_cast<uint32_t>(acc2[c * 32 + 16 + i] >> 32);
        }
        epi_write_row_256(bufs, lane, c, r0, r1, g.alpha);
      }
      direct_store_half<Cfg, Policy>(p, bufs, lane, q, h, 2, sub, m_blk, n_blk, tg, local_tile, lr);
      __syncwarp();
      if (Policy::kSignalPerTile && !local_tile) {
        if (lane == 0) {
          const uint32_t slot = seq & 7u;
          if (!mbar_wait(&ctl->sig_empty[slot], ((seq >> 3) & 1u) ^ 1u, &ctl->abort_flag, status,
                         0x800 + slot))
            return;
          mbar_arrive(&ctl->sig_full[slot]);
        }
        ++seq;
      }
    } else {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r0[32], r1[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          r0[2 * i] = static_cast<uint32_t>(acc2[c * 32 + i]);
          r0[2 * i + 1] = static_cast<uint32_t>(acc2[c * 32 + i] >> 32);
          r1[2 * i] = static_cast<uint32_t>(acc2[c * 32 + 16 + i]);
          r1[2 * i + 1] = static_cast<uint32_t>(acc2[c * 32 + 16 + i] >> 32);
        }
        // The buffer about to be filled was read by the store issued two boxes ago.
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
        uint8_t* b = bufs + sbuf * Cfg::EPI_BUF_BYTES;
        epi_write_row_swizzled(b, lane, r0, r1, g.alpha);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          Policy::store_box(p, m_blk, n_blk, sub * Cfg::CTA_M + static_cast<int>(q * 32u),
                            h * 128 + c * Cfg::EPI_COLS, b);
          bulk_commit();
        }
        sbuf ^= 1u;
      }
      if (lane == 0) Policy::tile_done(p, m_blk, n_blk, sub * 4 + static_cast<int>(q));
    }
  }
  if constexpr (!Policy::kDirect) {
    if (lane == 0) bulk_wait_all<0>();
  }
}

template <class Cfg, class Policy, class P>
__device__ __forceinline__ void gemm_epilogue(const P& p, const GemmShape& g, uint8_t* epi_smem,
                                              GemmCtl<Cfg::STAGES>* ctl, uint32_t* status,
                                              int cta, int num_ctas, uint32_t tmem_base,
                                              uint32_t warp, uint32_t lane, int sub) {
  if constexpr (Cfg::BS) {
    gemm_epilogue_bs<Cfg, Policy>(p, g, epi_smem, ctl, status, cta, num_ctas, tmem_base, warp, lane,
                                  sub);
  } else if constexpr (Policy::kDirect) {
    gemm_epilogue_direct<Cfg, Policy>(p, g, epi_smem, ctl, status, cta, num_ctas, tmem_base, warp,
                                      lane, sub);
  } else {
    gemm_epilogue_tma<Cfg, Policy>(p, g, epi_smem, ctl, status, cta, num_ctas, tmem_base, warp,
                                   lane, sub);
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
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->sf_full[i], 4 * Cfg::PAIR);  // one arrival per scale warp (of the pair)
      mbar_init(&ctl->sf_empty[i], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&ctl->tmem_full[a], 1);
      mbar_init(&ctl->tmem_empty[a], Cfg::EPI_WARPS * Cfg::PAIR);  // one arrival per epilogue warp (of the pair)
    }
    for (int i = 0; i < 8; ++i) {
      mbar_init(&ctl->sig_full[i], Cfg::EPI_WARPS);
      mbar_init(&ctl->sig_empty[i], 1);
    }
    ctl->abort_flag = 0;
    ctl->a_ready_tiles = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    if constexpr (Cfg::PAIR == 2) {
      tmem_alloc_pair(&ctl->tmem_base, Cfg::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&ctl->tmem_base, Cfg::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if constexpr (Cfg::PAIR == 2) {
    // The partner arrives on this CTA's barriers: they must be initialised before it starts.
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  tc_fence_after_sync();
  return *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
}

template <class Cfg>
__device__ __forceinline__ void gemm_teardown(GemmCtl<Cfg::STAGES>* ctl, uint32_t warp,
                                              uint32_t tmem_base) {
  tc_fence_before_sync();
  if constexpr (Cfg::PAIR == 2) {
    // A role that gave up tells the partner CTA, whose roles may still be waiting for it.
    __syncwarp();
    if ((threadIdx.x & 31u) == 0 && *reinterpret_cast<volatile int*>(&ctl->abort_flag) != 0)
      st_cluster_u32(map_to_cta(smem_u32(&ctl->abort_flag), cluster_ctarank() ^ 1u), 1u);
    // Nobody leaves while the partner may still arrive on this CTA's barriers or while the
    // even CTA's MMAs may still read this CTA's operand ring.
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  if (*reinterpret_cast<volatile int*>(&ctl->abort_flag) != 0) {
    // Some wait gave up: loads may still be landing in this CTA's shared memory.
    // Give them a bounded grace period before the CTA (and its memory) goes away.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    if constexpr (Cfg::PAIR == 2) cluster_sync_all();
    else __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    if constexpr (Cfg::PAIR == 2) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
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
  // A pair walks the tile list as one worker; `sub` is this CTA's half of every tile.
  const int sub = Cfg::PAIR == 2 ? static_cast<int>(cluster_ctarank()) : 0;
  const int worker = cta / Cfg::PAIR, num_workers = num_ctas / Cfg::PAIR;
  if constexpr (Cfg::BS) {
    // 128 x 56 + 256 x 224 registers = 64,512, what 384 threads x 168 were launched with.
    if (warp < 4) {
      warpgroup_reg_dec<56>();
      if (warp == 0) {
        gemm_producer<Cfg, Policy>(p, g, ring, &ctl, status, worker, num_workers, sub);
      } else if (warp == 1) {
        if (sub == 0)
          gemm_mma_bs<Cfg, Policy>(p, g, ring, &ctl, status, worker, num_workers, tmem_base);
      } else if (warp == 2) {
        if constexpr (Policy::kDirect && Policy::kSignalPerTile) {
          if (lane == 0) gemm_signal<Cfg, Policy>(p, &ctl, status, worker, num_workers, sub);
        }
      }
    } else {
      warpgroup_reg_inc<224>();
      gemm_epilogue<Cfg, Policy>(p, g, epi, &ctl, status, worker, num_workers, tmem_base, warp,
                                 lane, sub);
    }
  } else if (warp == 0) {
    gemm_producer<Cfg, Policy>(p, g, ring, &ctl, status, worker, num_workers, sub);
  } else if (warp == 1) {
    if constexpr (Cfg::MX) {
      if (sub == 0)
        gemm_mma_mx<Cfg, Policy>(p, g, ring, &ctl, status, worker, num_workers, tmem_base);
    } else {
      if (sub == 0)
        gemm_mma<Cfg, Policy>(p, g, ring, &ctl, status, worker, num_workers, tmem_base);
    }
  } else if (Cfg::MX && warp >= Cfg::SCALE_WARP0) {
    if constexpr (Cfg::MX)
      gemm_scale_writer<Cfg, Policy>(p, g, &ctl, status, worker, num_workers, tmem_base, warp,
                                     lane, sub);
  } else if (warp < 2 + Cfg::EPI_WARPS) {
    gemm_epilogue<Cfg, Policy>(p, g, epi, &ctl, status, worker, num_workers, tmem_base, warp,
                               lane, sub);
  } else if (warp == Cfg::SIGNAL_WARP) {
    if constexpr (Policy::kDirect && Policy::kSignalPerTile) {
      if (lane == 0) gemm_signal<Cfg, Policy>(p, &ctl, status, worker, num_workers, sub);
    }
  }
  __syncwarp();
  gemm_teardown<Cfg>(&ctl, warp, tmem_base);
}

}  // namespace cb
