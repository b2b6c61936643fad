// Fused GEMM -> reduce-scatter:
//   out[M/W, N] (rows of rank r) = sum over ranks q of  A_q[M, K_local] * B_q[N, K_local]^T
//
// ONE kernel per rank.  The tcgen05 GEMM walks the output row blocks owner by
// owner, starting with the next rank (so at any moment the W ranks write to W
// different owners) and ending with its OWN rows.  For another rank's rows the
// epilogue writes the bf16 partial tile straight into the owner's staging slot
// for this source rank (row-contiguous 16-byte stores over NVLink) and bumps a
// per-tile arrival counter there.  For its own rows - by then the other ranks'
// partials have had a whole owner-chunk of time to arrive - the epilogue waits
// for the tile's W-1 arrivals, adds the staged partials to its accumulator in
// fp32 in rank order and writes the final bf16 rows: the reduction runs under
// the main loop of the next tile, the local partial never goes through memory,
// and there is no reduction phase after the GEMM.  Deterministic (fixed order).
//
// The reference fuses the same pair with in-flight `store_add` into the
// owner's C (datasets/example054_thunderkitten_gemm_rs_easy/nv/
// empty_thunderkitten_gemm_rs.cu:141-208, task rotation at :112-139), i.e. bf16
// accumulation in arrival order plus a trailing barrier; here partials are
// kept apart and summed in fp32, and call-parity double buffering replaces the
// barrier.
#include "fused_common.cuh"

#include <string>

#include "../gemm/launch.h"
#include "../gemm/tmap_host.h"
#include "../symm/driver_api.h"

namespace cb {

static constexpr int kRsMaxTiles = 8192;  // flags per parity

struct GemmRsParams {
  CUtensorMap tm_a;
  CUtensorMap tm_b;
  uint8_t* stage_peer[2][CB_MAX_RANKS];  // [parity][owner]: owner's staging (all source slots)
  GemmShape g;
  int rank, world;
  int blocks_per_rank;  // row blocks (one tile height each) of the output owned by each rank
  int raster_group;
  const uint8_t* stage_local[2];  // my staging: [W sources][M/W][N] bf16
  uint32_t* flags_peer[CB_MAX_RANKS];  // [2][kRsMaxTiles] on each rank
  uint32_t* flags_local;
  void* out;  // [M/W, N] bf16
  FusedSeq seq;
  uint32_t* status;
  unsigned long long timeout_ns;
  unsigned int poll_ns;  // pause between polls of a tile's arrival counter
};

struct RsRt {
  const GemmRsParams* p;
  uint32_t parity;
};

template <class Cfg>
struct RsPolicy {
  __device__ static int num_tiles(const RsRt& r) {
    return r.p->g.num_m_blocks * r.p->g.num_n_blocks;
  }
  // tile -> (owner, local row block, column block); owners visited rank+1, rank+2, ..., rank.
  __device__ static void decode(const GemmRsParams& p, int tile, int* owner, int* lm, int* n) {
    const int per_owner = p.blocks_per_rank * p.g.num_n_blocks;
    const int oi = tile / per_owner;
    *owner = (p.rank + 1 + oi) % p.world;
    raster_tile(tile - oi * per_owner, p.blocks_per_rank, p.g.num_n_blocks, p.raster_group, lm, n);
  }
  __device__ static void tile_coord(const RsRt& r, int tile, int* m, int* n) {
    int owner, lm;
    decode(*r.p, tile, &owner, &lm, n);
    *m = owner * r.p->blocks_per_rank + lm;
  }
  __device__ static const CUtensorMap* map_a(const RsRt& r, int) { return &r.p->tm_a; }
  __device__ static const CUtensorMap* map_b(const RsRt& r) { return &r.p->tm_b; }
  __device__ static int a_row(const RsRt&, int m_blk) { return m_blk * Cfg::BM; }
  __device__ static bool wait_a_ready(const RsRt&, int, volatile int*) { return true; }
  static constexpr bool kDirect = true;
  static constexpr bool kSignalPerTile = true;
  static constexpr bool kScatterRows = false;
  static constexpr bool kReduceLocal = true;
  __device__ static int b_row(const RsRt&, int, int n_blk) { return n_blk * Cfg::BN; }
  __device__ static bool tile_is_local(const RsRt& r, int m_blk) {
    return m_blk / r.p->blocks_per_rank == r.p->rank;
  }
  // Arrival counter of the rows that CTA `sub` of a pair produces / consumes for local tile
  // (lm, n_blk).
  __device__ static int flag_index(const GemmRsParams& p, int lm, int n_blk, int sub) {
    return (lm * p.g.num_n_blocks + n_blk) * Cfg::PAIR + sub;
  }
  __device__ static bool wait_local_ready(const RsRt& r, int m_blk, int n_blk, int sub) {
    const GemmRsParams& p = *r.p;
    const int lm = m_blk - p.rank * p.blocks_per_rank;
    const uint32_t* f = p.flags_local + r.parity * kRsMaxTiles + flag_index(p, lm, n_blk, sub);
    return wait_flag_ge_sys_paced(f, static_cast<uint32_t>(p.world - 1), p.timeout_ns, p.status,
                                  PH_RS_TILE, lm * p.g.num_n_blocks + n_blk, p.poll_ns);
  }
  __device__ static void local_reduce(const RsRt& r, int m_blk, int n_blk, LocalReduce* t) {
    const GemmRsParams& p = *r.p;
    const int lm = m_blk - p.rank * p.blocks_per_rank;
    const long long Ml = p.g.M / p.world;
    const long long ld = static_cast<long long>(p.g.N) * 2;
    const long long tile_off =
        (static_cast<long long>(lm) * Cfg::BM * p.g.N + static_cast<long long>(n_blk) * Cfg::BN) *
        2;
    // Copies in rank order (own rank left out): the sum does not depend on timing.
    t->nsrc = p.world - 1;
#pragma unroll
    for (int i = 0; i < 7; ++i) {
      const int s = i + (i >= p.rank ? 1 : 0);
      t->src[i] = p.stage_local[r.parity] + static_cast<long long>(s) * Ml * ld + tile_off;
    }
    t->src_ld = ld;
    t->out = static_cast<uint8_t*>(p.out) + tile_off;
    t->out_ld = ld;
  }
  __device__ static void direct_targets(const RsRt& r, int m_blk, int n_blk, DirectTargets* t) {
    const GemmRsParams& p = *r.p;
    const int owner = m_blk / p.blocks_per_rank;
    const int lm = m_blk - owner * p.blocks_per_rank;
    const long long Ml = p.g.M / p.world;
    t->n = 1;
    t->ld_bytes = static_cast<long long>(p.g.N) * 2;
    t->base[0] = p.stage_peer[r.parity][owner] +
                 ((static_cast<long long>(p.rank) * Ml + lm * Cfg::BM) * p.g.N +
                  static_cast<long long>(n_blk) * Cfg::BN) * 2;
    t->rows = Cfg::BM;
    const int left = p.g.N - n_blk * Cfg::BN;
    t->cols = left < Cfg::BN ? left : Cfg::BN;
  }
  // Signal thread, after its release fence covered the tile's stores.
  __device__ static void tile_done(const RsRt& r, int m_blk, int n_blk, int quadrant) {
    const GemmRsParams& p = *r.p;
    const int owner = m_blk / p.blocks_per_rank;
    const int lm = m_blk - owner * p.blocks_per_rank;
    red_relaxed_sys_add(
        p.flags_peer[owner] + r.parity * kRsMaxTiles + flag_index(p, lm, n_blk, quadrant >> 2),
        1u);
  }
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
    gemm_rs_kernel(const __grid_constant__ GemmRsParams p0, const GemmRsParams* emu,
                   int ctas_per_rank) {
  extern __shared__ uint8_t smem_raw[];
  const int vrank = emu != nullptr ? blockIdx.x / ctas_per_rank : 0;
  const GemmRsParams& p = emu != nullptr ? emu[vrank] : p0;
  const int cta = blockIdx.x - vrank * ctas_per_rank;
  const uint32_t parity = fused_begin(p.seq);
  RsRt rt{&p, parity};
  gemm_cta_main<Cfg, RsPolicy<Cfg>>(rt, p.g, p.status, cta, ctas_per_rank, smem_raw);
  // Last CTA out clears this parity's arrival counters (every wait of this call is over by
  // then; the peers' next additions to them belong to the call after next).
  __syncthreads();
  __shared__ int last_cta;
  if (threadIdx.x == 0) {
    __threadfence();
    last_cta = atomicAdd(p.seq.done_ctas, 1u) == static_cast<uint32_t>(ctas_per_rank) - 1u;
  }
  __syncthreads();
  if (last_cta) {
    const int nflags = p.blocks_per_rank * p.g.num_n_blocks * Cfg::PAIR;
    for (int i = threadIdx.x; i < nflags; i += blockDim.x)
      p.flags_local[parity * kRsMaxTiles + i] = 0u;
    __syncthreads();
    if (threadIdx.x == 0) {
      *p.seq.done_ctas = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.seq.seq) = ld_volatile(p.seq.seq) + 1u;
    }
  }
}

template <class Cfg>
static int launch_rs(const GemmRsParams& p, const GemmRsParams* emu, int emu_world,
                     int ctas_per_rank, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(gemm_rs_kernel<Cfg>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    return -1;
  }
  if (ctas_per_rank % Cfg::PAIR != 0) {
    set_last_error("gemm_rs: the CTA count must be even for CTA-pair tiles");
    return -1;
  }
  const int grid = emu != nullptr ? ctas_per_rank * emu_world : ctas_per_rank;
  e = launch_gemm_kernel(gemm_rs_kernel<Cfg>, grid, Cfg::THREADS, Cfg::SMEM_BYTES, st, Cfg::PAIR,
                         emu != nullptr, p, emu, ctas_per_rank);
  if (e != cudaSuccess) {
    set_last_error(std::string("gemm_rs launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // namespace cb

using namespace cb;

extern "C" {

// Polls of a local tile's arrival counter are 3 us apart.  Measured on 4 GPUs at the bench
// shape, two sweeps: at 300 ns the CTAs that reach their own tiles early delay the peers'
// partial tiles on their way in (fp8 0.69 / 0.85 ms, bf16 0.67 / 1.04 ms); 1 us: 0.49 / 0.85
// and 0.67 / 0.88; 3 us: 0.376 / 0.374 and 0.65 / 0.68; 10 us: 0.44 / 0.41 and 0.69 / 0.65 (the
// waits themselves start to cost).  Run-to-run spread from the power state is of the same
// size as the smaller differences; the 300 ns -> 3 us step is not.
static unsigned int g_rs_poll_ns = 3000u;

struct CbGemmRsDesc {
  int rank, world;
  int M, N, K;            // K = local K shard
  int fp8;
  float alpha;
  int bn;                 // 256 or 128: one CTA per 128 x bn tile; 512: a CTA pair per 256 x 256
  int ctas_per_rank;
  const void* a;          // [M, K]
  const void* b;          // [N, K]
  void* out;              // [M/world, N] bf16
  void* stage_peer[2][CB_MAX_RANKS];  // staging [W][M/W][N] bf16 per parity and rank
  void* flags_peer[CB_MAX_RANKS];     // uint32 [2][8192] per rank
  void* seq;
  void* status;
  unsigned long long timeout_ns;
  // bn == 192 only (fp8 with power-of-two block scales, CTA pairs on 256 x 192 tiles): packed
  // exponent words, see cb_gemm_fp8_mx.
  const void* a_sf;   // [ceil(K/512)][M]
  const void* b_sf;   // [ceil(K/512)][N]
};

static int build_rs_params(const CbGemmRsDesc& d, GemmRsParams* p) {
  const int esz = d.fp8 ? 1 : 2;
  const int BK = d.fp8 ? 128 : 64;
  const TmapDtype dt = d.fp8 ? TMAP_U8 : TMAP_BF16;
  const bool mx = d.bn == 192;
  const int pair = (d.bn == 512 || mx) ? 2 : 1;
  const int bm = 128 * pair;
  const int tile_n = d.bn == 512 ? 256 : d.bn;
  if (mx && (!d.fp8 || d.K % 128 != 0 || d.a_sf == nullptr || d.b_sf == nullptr)) {
    set_last_error("gemm_rs: bn 192 is the block-scaled fp8 form: fp8 inputs, K % 128 == 0 and "
                   "scale words for A and B");
    return -1;
  }
  if (d.world < 1 || d.M % (d.world * bm) != 0) {
    set_last_error("gemm_rs: M must be a multiple of world * tile height (128, or 256 for bn 512)");
    return -1;
  }
  if (d.K % 16 != 0 || d.N % 8 != 0) {
    set_last_error("gemm_rs: K % 16 == 0 and N % 8 == 0 required");
    return -1;
  }
  const int Ml = d.M / d.world;
  const int num_n = (d.N + tile_n - 1) / tile_n;
  if ((Ml / bm) * num_n * pair > kRsMaxTiles) {
    set_last_error("gemm_rs: too many output tiles per rank");
    return -1;
  }
  if (make_tmap_2d(&p->tm_a, d.a, dt, d.K, d.M, (unsigned long long)d.K * esz, BK, 128, true))
    return -1;
  if (make_tmap_2d(&p->tm_b, d.b, dt, d.K, d.N, (unsigned long long)d.K * esz, BK, tile_n / pair,
                   true))
    return -1;
  for (int par = 0; par < 2; ++par) {
    for (int o = 0; o < CB_MAX_RANKS; ++o)
      p->stage_peer[par][o] = static_cast<uint8_t*>(d.stage_peer[par][o]);
    p->stage_local[par] = static_cast<const uint8_t*>(d.stage_peer[par][d.rank]);
  }
  p->g.M = d.M;
  p->g.N = d.N;
  p->g.K = d.K;
  p->g.num_m_blocks = d.M / bm;
  p->g.num_n_blocks = num_n;
  p->g.num_k_blocks = (d.K + BK - 1) / BK;
  p->g.alpha = d.alpha;
  p->g.sfa = mx ? static_cast<const uint32_t*>(d.a_sf) : nullptr;
  p->g.sfb = mx ? static_cast<const uint32_t*>(d.b_sf) : nullptr;
  p->g.sfa_rows = d.M;
  p->g.sfb_rows = d.N;
  p->rank = d.rank;
  p->world = d.world;
  p->blocks_per_rank = Ml / bm;
  p->raster_group = p->blocks_per_rank < 8 ? p->blocks_per_rank : 8;
  for (int r = 0; r < CB_MAX_RANKS; ++r) p->flags_peer[r] = static_cast<uint32_t*>(d.flags_peer[r]);
  p->flags_local = static_cast<uint32_t*>(d.flags_peer[d.rank]);
  p->out = d.out;
  p->seq.seq = static_cast<uint32_t*>(d.seq);
  p->seq.done_ctas = static_cast<uint32_t*>(d.seq) + 1;
  p->status = static_cast<uint32_t*>(d.status);
  p->timeout_ns = d.timeout_ns;
  p->poll_ns = g_rs_poll_ns;
  return 0;
}

// Nanoseconds between polls of a local tile's arrival counter (tuning).
void cb_gemm_rs_set_poll_ns(unsigned int ns) { g_rs_poll_ns = ns; }

int cb_sizeof_gemm_rs_params() { return static_cast<int>(sizeof(GemmRsParams)); }

int cb_gemm_rs(const CbGemmRsDesc* descs, int n, void* emu_table, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n < 1 || n > CB_MAX_RANKS) return -1;
  GemmRsParams hp[CB_MAX_RANKS];
  for (int i = 0; i < n; ++i)
    if (build_rs_params(descs[i], &hp[i]) != 0) return -1;
  const GemmRsParams* emu = nullptr;
  if (n > 1) {
    if (emu_table == nullptr) {
      set_last_error("gemm_rs: emulation needs a device table");
      return -1;
    }
    cudaError_t e = cudaMemcpyAsync(emu_table, hp, sizeof(GemmRsParams) * n,
                                    cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) {
      set_last_error(std::string("gemm_rs: table copy: ") + cudaGetErrorString(e));
      return -1;
    }
    cudaStreamSynchronize(st);
    emu = static_cast<const GemmRsParams*>(emu_table);
  }
  const CbGemmRsDesc& d = descs[0];
  if (d.fp8) {
    if (d.bn == 192)
      return launch_rs<GemmCfg<192, 6, true, 2, false, true>>(hp[0], emu, n, d.ctas_per_rank, st);
    if (d.bn == 512)
      return launch_rs<GemmCfg<256, 6, true, 2>>(hp[0], emu, n, d.ctas_per_rank, st);
    if (d.bn == 256) return launch_rs<GemmCfg<256, 4, true>>(hp[0], emu, n, d.ctas_per_rank, st);
    if (d.bn == 128) return launch_rs<GemmCfg<128, 6, true>>(hp[0], emu, n, d.ctas_per_rank, st);
  } else {
    if (d.bn == 512)
      return launch_rs<GemmCfg<256, 6, false, 2>>(hp[0], emu, n, d.ctas_per_rank, st);
    if (d.bn == 256) return launch_rs<GemmCfg<256, 4, false>>(hp[0], emu, n, d.ctas_per_rank, st);
    if (d.bn == 128) return launch_rs<GemmCfg<128, 6, false>>(hp[0], emu, n, d.ctas_per_rank, st);
  }
  set_last_error("gemm_rs: bn must be 128, 256 or 512");
  return -1;
}

}  // extern "C"
