// Fused all-gather -> GEMM:  C[M, N_local] = allgather_rows(A_local)[M, K] * B[N_local, K]^T
//
// ONE kernel per rank.  A few CTAs ("comm CTAs") push this rank's A rows into
// every peer's gathered buffer (16-byte stores over NVLink, or one multimem.st
// per vector through the switch) and raise a per-row-block flag on the peer; the other CTAs run the tcgen05 GEMM, doing the tiles of
// their own rows first (straight from A_local) and then, in arrival order, the
// tiles of remote rows as soon as the row block's flag is up.  Transfer and
// math overlap row block by row block.
//
// The reference has the same split -- comm SMs storing A chunks through the
// multicast address plus per-row-block barriers, compute SMs waiting on them
// (datasets/example051_thunderkitten_ag_gemm_easy/nv/empty_thunderkitten_ag_gemm.cu:118-238)
// -- with NUM_DEVICES fixed at 8 and a separate clean-up kernel; here the world
// size is a run-time value, buffers/flags are double-buffered by call parity so
// no clean-up launch and no cross-GPU barrier is needed, and operand loads are
// never cluster-multicast.
#include "fused_common.cuh"

#include <string>

#include "../gemm/launch.h"
#include "../gemm/tmap_host.h"
#include "../symm/driver_api.h"

namespace cb {

static constexpr int kAgMaxRowBlocks = 1024;  // flags per parity

struct AgGemmParams {
  CUtensorMap tm_a_local;
  CUtensorMap tm_a_full[2];
  CUtensorMap tm_b;
  CUtensorMap tm_c;
  GemmShape g;
  int rank, world;
  int blocks_per_rank;  // row blocks (one tile height each) of A owned by each rank
  int parts;            // independent pieces a row block is pushed in
  int num_comm_ctas;
  int raster_group;
  unsigned long long row_block_bytes;
  const uint8_t* a_local;
  uint8_t* a_full_peer[2][CB_MAX_RANKS];
  uint8_t* a_full_mc[2];
  uint32_t* flags_peer[CB_MAX_RANKS];  // [2][kAgMaxRowBlocks] on each rank
  uint32_t* flags_mc;
  uint32_t* flags_local;
  FusedSeq seq;
  uint32_t* status;
  unsigned long long timeout_ns;
  // Hardware block scales (fp8): packed exponent words of the local A rows [K groups][M / W]
  // and, per parity and rank, of the gathered rows [K groups][M]; K groups = ceil(K / 512).
  const uint32_t* a_sf_local;
  uint32_t* a_sf_full_peer[2][CB_MAX_RANKS];
  int sf_kgroups;
  // Optional gate on the LOCAL rows: word r / src_ready_rows of `src_ready` reaches
  // `src_ready_target` once local row r is in memory (a host-to-device copy still in flight
  // when the kernel starts publishes its progress there).  nullptr: the rows are all there.
  const uint32_t* src_ready;
  uint32_t src_ready_target;
  int src_ready_rows;
  int block_rows;  // rows of one row block (the tile height)
  int gate_group;  // row blocks per raster panel of the local tiles while gated
  unsigned int gate_poll_ns;
  unsigned int row_poll_ns;  // > 0: pause between polls of a remote row block's counter
};

// Waits until every row of local row block `rb` has landed (bounded).  Polls are 20 us apart:
// with one lane of each of 148 CTAs polling the word every 500 ns, the stream memory operations
// that write those words - and the host-to-device copy queued behind them - crawled (a 2.6 ms
// copy took 14-17 ms); at 4 us it still took 5-8 ms; at 20 us the copy runs at full speed and a
// gated 8192 x 28672 x 8192 GEMM ends 0.8 ms after its 2.6 ms copy (5.5 ms back to back).  A piece
// of the copy takes 80 us or more, so slow polls cost little.
__device__ __forceinline__ bool ag_src_wait(const AgGemmParams& p, int rb) {
  if (p.src_ready == nullptr) return true;
  const int last_row = (rb + 1) * p.block_rows - 1;
  return wait_flag_ge_sys_paced(p.src_ready + last_row / p.src_ready_rows, p.src_ready_target,
                                p.timeout_ns, p.status, PH_AG_ROWS, 0x4000u + rb, p.gate_poll_ns);
}

struct AgRt {
  const AgGemmParams* p;
  uint32_t parity;
};

template <class Cfg>
struct AgPolicy {
  __device__ static int num_tiles(const AgRt& r) {
    return r.p->g.num_m_blocks * r.p->g.num_n_blocks;
  }
  // Processing order: this rank's own row blocks first (all column blocks), then, for
  // rb = 0, 1, ..., row block rb of every peer (the order the pushes arrive in).  The
  // remote part is rasterised in panels of W-1 row blocks, i.e. one arrival wave each - but
  // never fewer than four: every panel streams all of B once, and with two ranks a one-block
  // panel re-read a 235 MB B sixteen times per call.
  __device__ static void tile_coord(const AgRt& r, int tile, int* m, int* n) {
    const AgGemmParams& p = *r.p;
    const int bpr = p.blocks_per_rank;
    const int local_tiles = bpr * p.g.num_n_blocks;
    int i;
    if (tile < local_tiles) {
      // Rows still arriving from the host: narrow panels, so that the math follows the copy.
      raster_tile(tile, bpr, p.g.num_n_blocks, p.src_ready != nullptr ? p.gate_group : bpr, &i, n);
      *m = p.rank * bpr + i;
    } else {
      raster_tile(tile - local_tiles, (p.world - 1) * bpr, p.g.num_n_blocks,
                  p.world - 1 < 4 ? 4 : p.world - 1, &i, n);
      const int rb = i / (p.world - 1);
      const int peer = (p.rank + 1 + i % (p.world - 1)) % p.world;
      *m = peer * bpr + rb;
    }
  }
  __device__ static bool is_local(const AgGemmParams& p, int m_blk) {
    return m_blk / p.blocks_per_rank == p.rank;
  }
  __device__ static const CUtensorMap* map_a(const AgRt& r, int m_blk) {
    return is_local(*r.p, m_blk) ? &r.p->tm_a_local : &r.p->tm_a_full[r.parity];
  }
  __device__ static const CUtensorMap* map_b(const AgRt& r) { return &r.p->tm_b; }
  __device__ static int a_row(const AgRt& r, int m_blk) {
    return is_local(*r.p, m_blk) ? (m_blk - r.p->rank * r.p->blocks_per_rank) * Cfg::BM
                                 : m_blk * Cfg::BM;
  }
  __device__ static bool wait_a_ready(const AgRt& r, int m_blk, volatile int* abort_flag) {
    const AgGemmParams& p = *r.p;
    if (is_local(p, m_blk)) {
      if (p.src_ready == nullptr) return true;
      if (!ag_src_wait(p, m_blk - p.rank * p.blocks_per_rank)) {
        *abort_flag = 1;
        return false;
      }
      fence_proxy_async();  // written by a copy engine; read by our TMA loads
      return true;
    }
    const uint32_t* f = p.flags_local + r.parity * kAgMaxRowBlocks + m_blk;
    const bool arrived =
        p.row_poll_ns > 0u
            ? wait_flag_ge_sys_paced(f, static_cast<uint32_t>(p.parts), p.timeout_ns, p.status,
                                     PH_AG_ROWS, m_blk, p.row_poll_ns)
            : wait_flag_ge_sys(f, static_cast<uint32_t>(p.parts), p.timeout_ns, p.status,
                               PH_AG_ROWS, m_blk);
    if (!arrived) {
      *abort_flag = 1;
      return false;
    }
    // The rows were written by a peer's bulk copies; our TMA load must see them.
    fence_proxy_async();
    return true;
  }
  // Scale words of a tile's A rows: this rank's own array, or the gathered one.
  __device__ static const uint32_t* a_sf(const AgRt& r, int m_blk, long long* pitch) {
    const AgGemmParams& p = *r.p;
    if (is_local(p, m_blk)) {
      *pitch = p.g.M / p.world;
      return p.a_sf_local + (m_blk - p.rank * p.blocks_per_rank) * Cfg::BM;
    }
    *pitch = p.g.M;
    return p.a_sf_full_peer[r.parity][p.rank] + m_blk * Cfg::BM;
  }
  static constexpr bool kDirect = false;  // C is local: TMA-store epilogue
  static constexpr bool kSignalPerTile = false;
  static constexpr bool kScatterRows = false;
  __device__ static int b_row(const AgRt&, int, int n_blk) { return n_blk * Cfg::BN; }
  __device__ static void store_box(const AgRt& r, int m_blk, int n_blk, int row, int col,
                                   const void* smem_box) {
    tma_store_2d(&r.p->tm_c, smem_box, n_blk * Cfg::BN + col, m_blk * Cfg::BM + row);
  }
  __device__ static void tile_done(const AgRt&, int, int, int) {}
};

// Comm CTA: all threads stream pieces of the local A rows to every peer with
// 16-byte loads and stores (one multimem.st per vector when a multicast object is
// bound, W-1 plain peer stores otherwise), then bump the row block's flag on the
// peers.  Load/store traffic from a handful of CTAs saturates NVLink here, which
// bulk (TMA) copies issued from the same number of SMs did not.
__device__ __forceinline__ void ag_comm_cta(const AgGemmParams& p, uint32_t parity, int comm_cta) {
  // A row block (a multiple of 16 bytes) is cut into `parts` nearly equal runs of 16-byte
  // vectors; with parts == number of comm CTAs all of them work on the same row block, so
  // row blocks complete one after the other, in the order the compute CTAs want them.
  const unsigned long long rb_vecs = p.row_block_bytes / 16ull;
  const unsigned long long per_part = (rb_vecs + p.parts - 1) / p.parts;
  const bool use_mc = p.a_full_mc[parity] != nullptr && p.flags_mc != nullptr;
  for (int item = comm_cta; item < p.blocks_per_rank * p.parts; item += p.num_comm_ctas) {
    const int rb = item / p.parts;
    const int part = item % p.parts;
    if (p.src_ready != nullptr) {
      // A time-out is recorded in the status word; the CTA carries on (bounded) either way.
      if (threadIdx.x == 0) (void)ag_src_wait(p, rb);
      __syncthreads();
    }
    unsigned long long v_begin = per_part * part, v_end = v_begin + per_part;
    if (v_begin > rb_vecs) v_begin = rb_vecs;
    if (v_end > rb_vecs) v_end = rb_vecs;
    const unsigned long long piece_vecs = v_end - v_begin;
    const uint4* src = reinterpret_cast<const uint4*>(p.a_local + rb * p.row_block_bytes) + v_begin;
    const unsigned long long dst_vec =
        static_cast<unsigned long long>(p.rank * p.blocks_per_rank + rb) * rb_vecs + v_begin;
    const unsigned long long T = blockDim.x;
    unsigned long long i = threadIdx.x;
    if (use_mc) {
      uint4* mc = reinterpret_cast<uint4*>(p.a_full_mc[parity]) + dst_vec;
      for (; i + 7ull * T < piece_vecs; i += 8ull * T) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = ld_nc_v4(src + i + u * T);
#pragma unroll
        for (int u = 0; u < 8; ++u) mm_st_v4(mc + i + u * T, v[u]);
      }
      for (; i < piece_vecs; i += T) mm_st_v4(mc + i, ld_nc_v4(src + i));
    } else {
      for (; i + 1ull * T < piece_vecs; i += 2ull * T) {
        const uint4 v0 = ld_nc_v4(src + i), v1 = ld_nc_v4(src + i + T);
        for (int d = 1; d < p.world; ++d) {
          uint4* dst =
              reinterpret_cast<uint4*>(p.a_full_peer[parity][(p.rank + d) % p.world]) + dst_vec;
          st_sys_v4(dst + i, v0);
          st_sys_v4(dst + i + T, v1);
        }
      }
      for (; i < piece_vecs; i += T) {
        const uint4 v = ld_nc_v4(src + i);
        for (int d = 1; d < p.world; ++d)
          st_sys_v4(reinterpret_cast<uint4*>(p.a_full_peer[parity][(p.rank + d) % p.world]) +
                        dst_vec + i, v);
      }
    }
    // Block-scaled operands: the row block's scale words travel with its first piece.
    if (p.a_sf_local != nullptr && part == 0) {
      const int bm = static_cast<int>(p.row_block_bytes / (static_cast<unsigned long long>(p.g.K)));
      const int Ml = p.g.M / p.world;
      for (int w = threadIdx.x; w < p.sf_kgroups * bm; w += blockDim.x) {
        const int kg = w / bm, rr = w - kg * bm;
        const uint32_t v = p.a_sf_local[static_cast<long long>(kg) * Ml + rb * bm + rr];
        const long long dst = static_cast<long long>(kg) * p.g.M +
                              (p.rank * p.blocks_per_rank + rb) * bm + rr;
        for (int d = 1; d < p.world; ++d)
          st_relaxed_sys(p.a_sf_full_peer[parity][(p.rank + d) % p.world] + dst, v);
      }
    }
    // One thread fences for the CTA (the barrier makes the others' stores precede it);
    // the other warps go straight on to the next piece while that fence drains.
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_acq_rel_sys();
      const int m_blk = p.rank * p.blocks_per_rank + rb;
      if (use_mc) {
        mm_red_add_relaxed_u32(p.flags_mc + parity * kAgMaxRowBlocks + m_blk, 1u);
      } else {
        for (int d = 1; d < p.world; ++d)
          red_relaxed_sys_add(
              p.flags_peer[(p.rank + d) % p.world] + parity * kAgMaxRowBlocks + m_blk, 1u);
      }
    }
  }
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
    ag_gemm_kernel(const __grid_constant__ AgGemmParams p0, const AgGemmParams* emu,
                   int ctas_per_rank) {
  extern __shared__ uint8_t smem_raw[];
  const int vrank = emu != nullptr ? blockIdx.x / ctas_per_rank : 0;
  const AgGemmParams& p = emu != nullptr ? emu[vrank] : p0;
  const int cta = blockIdx.x - vrank * ctas_per_rank;
  const uint32_t parity = fused_begin(p.seq);
  const int ncomp = ctas_per_rank - p.num_comm_ctas;
  if (cta >= ncomp) {
    ag_comm_cta(p, parity, cta - ncomp);
  } else {
    AgRt rt{&p, parity};
    gemm_cta_main<Cfg, AgPolicy<Cfg>>(rt, p.g, p.status, cta, ncomp, smem_raw);
  }
  __syncthreads();
  // Last CTA out zeroes this parity's flags (all waits of this call are over by then).
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(p.seq.done_ctas, 1u);
    if (prev == static_cast<uint32_t>(ctas_per_rank) - 1u) {
      for (int m = 0; m < p.g.num_m_blocks; ++m)
        p.flags_local[parity * kAgMaxRowBlocks + m] = 0u;
      *p.seq.done_ctas = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.seq.seq) = ld_volatile(p.seq.seq) + 1u;
    }
  }
}

template <class Cfg>
static int launch_ag(const AgGemmParams& p, const AgGemmParams* emu, int emu_world,
                     int ctas_per_rank, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(ag_gemm_kernel<Cfg>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    return -1;
  }
  if (ctas_per_rank % Cfg::PAIR != 0 || p.num_comm_ctas % Cfg::PAIR != 0) {
    set_last_error("ag_gemm: CTA counts must be even for CTA-pair tiles");
    return -1;
  }
  // Emulated ranks wait on one another inside the launch: cooperative, so that all their
  // CTAs are resident together.
  const int grid = emu != nullptr ? ctas_per_rank * emu_world : ctas_per_rank;
  e = launch_gemm_kernel(ag_gemm_kernel<Cfg>, grid, Cfg::THREADS, Cfg::SMEM_BYTES, st, Cfg::PAIR,
                         emu != nullptr, p, emu, ctas_per_rank);
  if (e != cudaSuccess) {
    set_last_error(std::string("ag_gemm launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // namespace cb

using namespace cb;

extern "C" {

// Host-side description of one rank's call; pointers are device addresses.
struct CbAgGemmDesc {
  int rank, world;
  int M, N, K;            // M = rows of the gathered A (all ranks), N = local columns
  int fp8;                // 0 bf16, 1 fp8 e4m3 (inputs); output is bf16
  float alpha;
  int bn;                 // 256 or 128: one CTA per 128 x bn tile; 512: a CTA pair per 256 x 256
  int num_comm_ctas;      // 0 when world == 1
  int parts;              // pieces a row block is pushed in (0 < parts <= 1024)
  int ctas_per_rank;      // CTAs this rank's launch (or grid slice) uses
  const void* a_local;    // [M/world, K]
  const void* b;          // [N, K]
  void* c;                // [M, N] bf16
  void* a_full_peer[2][CB_MAX_RANKS];  // gathered buffers [M, K], per parity and rank
  void* a_full_mc[2];
  void* flags_peer[CB_MAX_RANKS];      // uint32 [2][1024] per rank
  void* flags_mc;
  void* seq;              // uint32 [2] local: {call counter, done CTAs}
  void* status;
  unsigned long long timeout_ns;
  // bn == 192 only (fp8 with power-of-two block scales applied by the tensor core, CTA pairs on
  // 256 x 192 tiles): packed exponent words, see cb_gemm_fp8_mx.
  const void* a_sf_local;                 // [ceil(K/512)][M / world]
  void* a_sf_full_peer[2][CB_MAX_RANKS];  // [ceil(K/512)][M] per parity and rank
  const void* b_sf;                       // [ceil(K/512)][N]
  // Optional: uint32 words that reach `src_ready_target` as the local rows land, one word per
  // `src_ready_rows` rows (nullptr: a_local is complete when the kernel starts).
  const void* src_ready;
  unsigned int src_ready_target;
  int src_ready_rows;
};

static unsigned int g_gate_poll_ns = 20000u;
static unsigned int g_row_poll_ns = 0u;

static int build_ag_params(const CbAgGemmDesc& d, AgGemmParams* p) {
  const int esz = d.fp8 ? 1 : 2;
  const int BK = d.fp8 ? 128 : 64;
  const TmapDtype dt = d.fp8 ? TMAP_U8 : TMAP_BF16;
  const bool mx = d.bn == 192;
  const int pair = (d.bn == 512 || mx) ? 2 : 1;
  const int bm = 128 * pair;                 // tile height = rows per flag
  const int tile_n = d.bn == 512 ? 256 : d.bn;
  if (mx && (!d.fp8 || d.K % 128 != 0 || d.a_sf_local == nullptr || d.b_sf == nullptr ||
             (d.world > 1 && d.a_sf_full_peer[0][d.rank] == nullptr))) {
    set_last_error("ag_gemm: bn 192 is the block-scaled fp8 form: fp8 inputs, K % 128 == 0 and "
                   "scale words for A (local and gathered) and B");
    return -1;
  }
  if (d.world < 1 || d.M % (d.world * bm) != 0) {
    set_last_error("ag_gemm: M must be a multiple of world * tile height (128, or 256 for bn 512)");
    return -1;
  }
  if (d.K % 16 != 0 || d.N % 8 != 0) {
    set_last_error("ag_gemm: K % 16 == 0 and N % 8 == 0 required");
    return -1;
  }
  if (d.M / bm > kAgMaxRowBlocks) {
    set_last_error("ag_gemm: too many row blocks");
    return -1;
  }
  if (d.parts < 1 || d.parts > 1024) {
    set_last_error("ag_gemm: parts must be in [1, 1024]");
    return -1;
  }
  const int Ml = d.M / d.world;
  if (make_tmap_2d(&p->tm_a_local, d.a_local, dt, d.K, Ml, (unsigned long long)d.K * esz, BK, 128,
                   true))
    return -1;
  for (int par = 0; par < 2; ++par) {
    const void* base = d.a_full_peer[par][d.rank];
    if (d.world > 1) {
      if (make_tmap_2d(&p->tm_a_full[par], base, dt, d.K, d.M, (unsigned long long)d.K * esz, BK,
                       128, true))
        return -1;
    } else {
      p->tm_a_full[par] = p->tm_a_local;
    }
  }
  if (make_tmap_2d(&p->tm_b, d.b, dt, d.K, d.N, (unsigned long long)d.K * esz, BK, tile_n / pair,
                   true))
    return -1;
  if (make_tmap_2d(&p->tm_c, d.c, TMAP_BF16, d.N, d.M, (unsigned long long)d.N * 2, 64, 32, true))
    return -1;
  p->g.M = d.M;
  p->g.N = d.N;
  p->g.K = d.K;
  p->g.num_m_blocks = d.M / bm;
  p->g.num_n_blocks = (d.N + tile_n - 1) / tile_n;
  p->g.num_k_blocks = (d.K + BK - 1) / BK;
  p->g.alpha = d.alpha;
  p->rank = d.rank;
  p->world = d.world;
  p->blocks_per_rank = Ml / bm;
  p->parts = d.parts;
  p->num_comm_ctas = d.world > 1 ? d.num_comm_ctas : 0;
  p->raster_group = p->blocks_per_rank < 8 ? p->blocks_per_rank : 8;
  p->row_block_bytes = static_cast<unsigned long long>(bm) * d.K * esz;
  p->a_local = static_cast<const uint8_t*>(d.a_local);
  for (int par = 0; par < 2; ++par) {
    for (int r = 0; r < CB_MAX_RANKS; ++r)
      p->a_full_peer[par][r] = static_cast<uint8_t*>(d.a_full_peer[par][r]);
    p->a_full_mc[par] = static_cast<uint8_t*>(d.a_full_mc[par]);
  }
  for (int r = 0; r < CB_MAX_RANKS; ++r) p->flags_peer[r] = static_cast<uint32_t*>(d.flags_peer[r]);
  p->flags_mc = static_cast<uint32_t*>(d.flags_mc);
  p->flags_local = static_cast<uint32_t*>(d.flags_peer[d.rank]);
  p->seq.seq = static_cast<uint32_t*>(d.seq);
  p->seq.done_ctas = static_cast<uint32_t*>(d.seq) + 1;
  p->status = static_cast<uint32_t*>(d.status);
  p->timeout_ns = d.timeout_ns;
  p->block_rows = bm;
  {
    // Every panel of local row blocks streams all of B once.  B that fits in L2 (126 MB) can be
    // walked one row block at a time; a larger B gets wider panels so that its re-reads stay a
    // small fraction of the HBM bandwidth (one row block at a time and a 470 MB B was 15 GB of
    // reads per GEMM).
    const double b_mb = static_cast<double>(d.N) * d.K * esz / (1 << 20);
    int gg = b_mb <= 96.0 ? 1 : (b_mb <= 256.0 ? 2 : 4);
    if (gg > p->blocks_per_rank) gg = p->blocks_per_rank;
    p->gate_group = gg;
  }
  p->gate_poll_ns = g_gate_poll_ns;
  p->row_poll_ns = g_row_poll_ns;
  p->src_ready = static_cast<const uint32_t*>(d.src_ready);
  p->src_ready_target = d.src_ready_target;
  p->src_ready_rows = d.src_ready_rows > 0 ? d.src_ready_rows : bm;
  if (d.src_ready != nullptr && d.src_ready_rows < 1) {
    set_last_error("ag_gemm: src_ready needs src_ready_rows >= 1");
    return -1;
  }
  p->a_sf_local = mx ? static_cast<const uint32_t*>(d.a_sf_local) : nullptr;
  for (int par = 0; par < 2; ++par)
    for (int r = 0; r < CB_MAX_RANKS; ++r)
      p->a_sf_full_peer[par][r] = mx ? static_cast<uint32_t*>(d.a_sf_full_peer[par][r]) : nullptr;
  p->sf_kgroups = (d.K / 128 + 3) / 4;
  p->g.sfb = mx ? static_cast<const uint32_t*>(d.b_sf) : nullptr;
  p->g.sfb_rows = d.N;
  if (d.world > 1 && p->num_comm_ctas < 1) {
    set_last_error("ag_gemm: world > 1 needs at least one comm CTA");
    return -1;
  }
  if (d.ctas_per_rank - p->num_comm_ctas < 1) {
    set_last_error("ag_gemm: no compute CTAs left");
    return -1;
  }
  return 0;
}

// Nanoseconds between polls of a remote row block's arrival counter (tuning; 0 = a few
// back-to-back polls, then 128 ns / 512 ns / 1 us apart).
void cb_ag_gemm_set_row_poll_ns(unsigned int ns) { g_row_poll_ns = ns; }

// Nanoseconds between polls of the local-rows gate (tuning; default 20000).
void cb_ag_gemm_set_gate_poll_ns(unsigned int ns) { g_gate_poll_ns = ns; }

int cb_sizeof_ag_gemm_params() { return static_cast<int>(sizeof(AgGemmParams)); }

// descs: `n` descriptors; n == 1 is a real rank, n > 1 emulates n ranks in one
// cooperative launch on the current device (`emu_table` = device buffer of
// n * cb_sizeof_ag_gemm_params() bytes that the call fills).
int cb_ag_gemm(const CbAgGemmDesc* descs, int n, void* emu_table, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n < 1 || n > CB_MAX_RANKS) return -1;
  AgGemmParams hp[CB_MAX_RANKS];
  for (int i = 0; i < n; ++i)
    if (build_ag_params(descs[i], &hp[i]) != 0) return -1;
  const AgGemmParams* emu = nullptr;
  if (n > 1) {
    if (emu_table == nullptr) {
      set_last_error("ag_gemm: emulation needs a device table");
      return -1;
    }
    cudaError_t e = cudaMemcpyAsync(emu_table, hp, sizeof(AgGemmParams) * n,
                                    cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) {
      set_last_error(std::string("ag_gemm: table copy: ") + cudaGetErrorString(e));
      return -1;
    }
    // hp lives on this stack frame: make sure the copy has read it.
    cudaStreamSynchronize(st);
    emu = static_cast<const AgGemmParams*>(emu_table);
  }
  const CbAgGemmDesc& d = descs[0];
  if (d.fp8) {
    if (d.bn == 192)
      return launch_ag<GemmCfg<192, 6, true, 2, false, true>>(hp[0], emu, n, d.ctas_per_rank, st);
    if (d.bn == 512)
      return launch_ag<GemmCfg<256, 6, true, 2>>(hp[0], emu, n, d.ctas_per_rank, st);
    if (d.bn == 256) return launch_ag<GemmCfg<256, 4, true>>(hp[0], emu, n, d.ctas_per_rank, st);
    if (d.bn == 128) return launch_ag<GemmCfg<128, 6, true>>(hp[0], emu, n, d.ctas_per_rank, st);
  } else {
    if (d.bn == 512)
      return launch_ag<GemmCfg<256, 6, false, 2>>(hp[0], emu, n, d.ctas_per_rank, st);
    if (d.bn == 256) return launch_ag<GemmCfg<256, 4, false>>(hp[0], emu, n, d.ctas_per_rank, st);
    if (d.bn == 128) return launch_ag<GemmCfg<128, 6, false>>(hp[0], emu, n, d.ctas_per_rank, st);
  }
  set_last_error("ag_gemm: bn must be 128, 256 or 512");
  return -1;
}

}  // extern "C"
