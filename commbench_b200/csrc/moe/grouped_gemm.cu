// Grouped (per-expert) tcgen05 GEMMs over the expert-major receive buffer.
//
//   up:    H1[rows, 2I] = A[rows, H] * W1[e][2I, H]^T          (TMA-store epilogue, local)
//          or, gated: S[rows, I] = silu(A * Wgate^T) * (A * Wup^T) in the same epilogue
//   down:  O[rows, H]   = S[rows, I] * W2[e][H, I]^T, each output row written straight
//          into the combine buffer of the rank that owns the token (fused combine send)
//
// Rows are grouped by local expert, every group padded to a multiple of 128, so
// one 128-row block belongs to exactly one expert: `mblk_expert[m_blk]` picks the
// weight slab, the number of row blocks is read from device memory (it depends
// on the routing), and the tile list is simply (row block, column block).
//
// The reference's grouped GEMM for the same layer is a scalar-FMA kernel
// (datasets/example056_thunderkitten_moe_dispatch_gemm_easy/nv/
// empty_thunderkitten_moe_dispatch_gemm.cu:227-293); its combine sends expert
// outputs back in a separate kernel (datasets/example082_deepep_jit_combine/nv/
// empty_deepep_jit_combine.cu:15-67).
#include "../gemm/gemm_sm100.cuh"

#include <string>

#include "../gemm/tmap_host.h"
#include "../prim/barrier.cuh"
#include "../symm/driver_api.h"

namespace cb {

struct GroupedParams {
  CUtensorMap tm_a;   // [max_rows, K]
  CUtensorMap tm_b;   // [E_local * N, K]   (expert slabs stacked along rows)
  CUtensorMap tm_c;   // [max_rows, N]      (up projection only)
  GemmShape g;        // M = max_rows (upper bound), N, K
  const int* mblk_expert;  // [max_rows / 128]
  const int* n_mblocks;    // device word: row blocks in use
  // down projection: scatter to token owners
  const int2* recv_meta;               // [max_rows] {owner rank, pair index} or {-1,-1}
  uint8_t* combine_peer[CB_MAX_RANKS]; // owner's combine buffer [T*K, N] bf16
  uint32_t* done_peer[CB_MAX_RANKS];   // owner's done words [W]
  uint32_t* done_ctas;                 // local scratch counter
  int rank, world;
  uint32_t* status;
};

// kGatedUp (up projection only): the weight slab of every expert is stored with its rows
// interleaved per column block - 128 gate rows, then the 128 up rows of the same outputs - and
// the epilogue writes silu(gate) * up, [rows, N/2], so H1 never exists in memory.
template <class Cfg, bool kDown, bool kGatedUp = false>
struct GroupedPolicy {
  using P = GroupedParams;
  static constexpr bool kGated = kGatedUp;
  static_assert(!(kDown && kGatedUp), "the gated epilogue belongs to the up projection");
  __device__ static int num_tiles(const P& p) {
    int mb = *reinterpret_cast<const volatile int*>(p.n_mblocks);
    if (mb > p.g.num_m_blocks) mb = p.g.num_m_blocks;
    return mb * p.g.num_n_blocks;
  }
  // Column blocks of one row block run together: the A row block is read once
  // from HBM and the expert's weight slab stays in L2 across the expert's row blocks.
  __device__ static void tile_coord(const P& p, int tile, int* m, int* n) {
    *m = tile / p.g.num_n_blocks;
    *n = tile - *m * p.g.num_n_blocks;
  }
  __device__ static const CUtensorMap* map_a(const P& p, int) { return &p.tm_a; }
  __device__ static const CUtensorMap* map_b(const P& p) { return &p.tm_b; }
  __device__ static int a_row(const P&, int m_blk) { return m_blk * Cfg::BM; }
  __device__ static int b_row(const P& p, int m_blk, int n_blk) {
    return p.mblk_expert[m_blk] * p.g.N + n_blk * Cfg::BN;
  }
  __device__ static bool wait_a_ready(const P&, int, volatile int*) { return true; }
  static constexpr bool kDirect = kDown;
  static constexpr bool kSignalPerTile = false;  // one completion flag per kernel instead
  static constexpr bool kScatterRows = kDown;
  __device__ static void store_box(const P& p, int m_blk, int n_blk, int row, int col,
                                   const void* smem_box) {
    tma_store_2d(&p.tm_c, smem_box, n_blk * (kGatedUp ? Cfg::BN / 2 : Cfg::BN) + col,
                 m_blk * Cfg::BM + row);
  }
  __device__ static void direct_targets(const P&, int, int, DirectTargets* t) {
    t->n = 0;
    t->ld_bytes = 0;
    t->rows = Cfg::BM;
    t->cols = Cfg::BN;
  }
  // Destination of output row `row` of row block m_blk: the owner's combine slot, or null
  // for padding rows.
  __device__ static uint8_t* row_base(const P& p, int m_blk, int row) {
    const int2 m = p.recv_meta[static_cast<long long>(m_blk) * Cfg::BM + row];
    if (m.x < 0) return nullptr;
    return p.combine_peer[m.x] + static_cast<long long>(m.y) * p.g.N * 2;
  }
  __device__ static void tile_done(const P&, int, int, int) {}
};

template <class Cfg, bool kDown, bool kGatedUp>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
    grouped_gemm_kernel(const __grid_constant__ GroupedParams p) {
  extern __shared__ uint8_t smem_raw[];
  gemm_cta_main<Cfg, GroupedPolicy<Cfg, kDown, kGatedUp>>(p, p.g, p.status, blockIdx.x, gridDim.x,
                                                          smem_raw);
  if constexpr (kDown) {
    // Every CTA releases its rows; the last one tells every owner that this expert rank
    // is done (the owners' combine reduction waits for W such words).
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_acq_rel_sys();
      if (atomicAdd(p.done_ctas, 1u) == gridDim.x - 1) {
        *p.done_ctas = 0u;
        fence_acq_rel_sys();
        for (int d = 0; d < p.world; ++d) {
          const int dest = (p.rank + d) % p.world;
          red_relaxed_sys_add(p.done_peer[dest] + p.rank, 1u);
        }
      }
    }
  }
}

template <class Cfg, bool kDown, bool kGatedUp = false>
static int launch_grouped(const GroupedParams& p, int ctas, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<Cfg, kDown, kGatedUp>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    return -1;
  }
  grouped_gemm_kernel<Cfg, kDown, kGatedUp><<<ctas, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(std::string("grouped gemm launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // namespace cb

using namespace cb;

extern "C" {

struct CbGroupedDesc {
  int max_rows, N, K, n_local_experts;
  int down;          // 0: up projection (C local), 1: down projection with combine scatter
  int rank, world;
  int ctas;
  int gated;         // up only: b is gate/up interleaved per 256 rows, c = silu(gate) * up
  const void* a;     // [max_rows, K] bf16
  const void* b;     // [n_local_experts * N, K] bf16
  void* c;           // up only: [max_rows, N] bf16, or [max_rows, N / 2] when gated
  const void* mblk_expert;
  const void* n_mblocks;
  const void* recv_meta;
  void* combine_peer[CB_MAX_RANKS];
  void* done_peer[CB_MAX_RANKS];
  void* done_ctas;
  void* status;
};

int cb_moe_grouped_gemm(const CbGroupedDesc* d, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  using Cfg = GemmCfg<256, 4, false>;
  if (d->max_rows % 128 != 0 || d->K % 8 != 0 || d->N % Cfg::BN != 0) {
    set_last_error("grouped gemm: max_rows % 128 == 0, K % 8 == 0, N % 256 == 0 required");
    return -1;
  }
  GroupedParams p;
  if (make_tmap_2d(&p.tm_a, d->a, TMAP_BF16, d->K, d->max_rows, (unsigned long long)d->K * 2,
                   Cfg::BK, Cfg::BM, true))
    return -1;
  if (make_tmap_2d(&p.tm_b, d->b, TMAP_BF16, d->K, (unsigned long long)d->n_local_experts * d->N,
                   (unsigned long long)d->K * 2, Cfg::BK, Cfg::BN, true))
    return -1;
  if (d->gated && d->down) {
    set_last_error("grouped gemm: the gated epilogue belongs to the up projection");
    return -1;
  }
  if (!d->down) {
    const unsigned long long c_cols = d->gated ? d->N / 2 : d->N;
    if (make_tmap_2d(&p.tm_c, d->c, TMAP_BF16, c_cols, d->max_rows, c_cols * 2, Cfg::EPI_COLS, 32,
                     true))
      return -1;
  } else {
    p.tm_c = p.tm_a;
  }
  p.g.M = d->max_rows;
  p.g.N = d->N;
  p.g.K = d->K;
  p.g.num_m_blocks = d->max_rows / 128;
  p.g.num_n_blocks = d->N / Cfg::BN;
  p.g.num_k_blocks = (d->K + Cfg::BK - 1) / Cfg::BK;
  p.g.alpha = 1.0f;
  p.mblk_expert = static_cast<const int*>(d->mblk_expert);
  p.n_mblocks = static_cast<const int*>(d->n_mblocks);
  p.recv_meta = static_cast<const int2*>(d->recv_meta);
  for (int r = 0; r < CB_MAX_RANKS; ++r) {
    p.combine_peer[r] = static_cast<uint8_t*>(d->combine_peer[r]);
    p.done_peer[r] = static_cast<uint32_t*>(d->done_peer[r]);
  }
  p.done_ctas = static_cast<uint32_t*>(d->done_ctas);
  p.rank = d->rank;
  p.world = d->world;
  p.status = static_cast<uint32_t*>(d->status);
  int ctas = d->ctas > 0 ? d->ctas : 148;
  if (d->down) return launch_grouped<Cfg, true>(p, ctas, st);
  return d->gated ? launch_grouped<Cfg, false, true>(p, ctas, st)
                  : launch_grouped<Cfg, false, false>(p, ctas, st);
}

}  // extern "C"
