// Fused GEMM -> reduce-scatter:
//   out[M/W, N] (rows of rank r) = sum over ranks q of  A_q[M, K_local] * B_q[N, K_local]^T
//
// ONE kernel per rank.  The tcgen05 GEMM walks the output row blocks owner by
// owner, starting with the next rank (so at any moment the W ranks write to W
// different owners); the epilogue writes each bf16 partial tile straight into
// the OWNER's staging slot for this source rank (row-contiguous 16-byte stores
// over NVLink) and bumps a per-tile arrival counter there.  When a CTA has finished its GEMM tiles it turns to the
// reduction of this rank's own output tiles: wait until all W partials of a
// tile arrived, add them in fp32, write bf16.  The transfer of tile i overlaps
// the math of tile i+1; the result is deterministic (fixed summation order).
//
// The reference fuses the same pair with in-flight `store_add` into the
// owner's C (datasets/example054_thunderkitten_gemm_rs_easy/nv/
// empty_thunderkitten_gemm_rs.cu:141-208, task rotation at :112-139), i.e. bf16
// accumulation in arrival order plus a trailing barrier; here partials are
// kept apart and summed in fp32, and call-parity double buffering replaces the
// barrier.
#include "fused_common.cuh"

#include <string>

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
  int blocks_per_rank;  // 128-row blocks of the output owned by each rank
  int raster_group;
  const uint8_t* stage_local[2];  // my staging: [W sources][M/W][N] bf16
  uint32_t* flags_peer[CB_MAX_RANKS];  // [2][kRsMaxTiles] on each rank
  uint32_t* flags_local;
  void* out;  // [M/W, N] bf16
  FusedSeq seq;
  uint32_t* status;
  unsigned long long timeout_ns;
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
  __device__ static int b_row(const RsRt&, int, int n_blk) { return n_blk * Cfg::BN; }
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
  __device__ static void tile_done(const RsRt& r, int m_blk, int n_blk, int) {
    const GemmRsParams& p = *r.p;
    const int owner = m_blk / p.blocks_per_rank;
    const int lm = m_blk - owner * p.blocks_per_rank;
    red_relaxed_sys_add(
        p.flags_peer[owner] + r.parity * kRsMaxTiles + lm * p.g.num_n_blocks + n_blk, 1u);
  }
};

// Reduction of this rank's output tiles; all threads of the CTA take part.
template <class Cfg>
__device__ __forceinline__ void rs_reduce_phase(const GemmRsParams& p, uint32_t parity, int cta,
                                                int num_ctas) {
  const int Ml = p.g.M / p.world;
  const int ntiles = p.blocks_per_rank * p.g.num_n_blocks;
  constexpr int VPR = Cfg::BN / 8;  // 16-byte vectors per tile row
  const uint4* stage = reinterpret_cast<const uint4*>(p.stage_local[parity]);
  uint4* out = static_cast<uint4*>(p.out);
  const unsigned long long row_vecs = static_cast<unsigned long long>(p.g.N) / 8ull;
  for (int t = cta; t < ntiles; t += num_ctas) {
    const int lm = t / p.g.num_n_blocks;
    const int n_blk = t - lm * p.g.num_n_blocks;
    uint32_t* flag = p.flags_local + parity * kRsMaxTiles + t;
    bool ok = true;
    if (threadIdx.x == 0)
      ok = wait_flag_ge_sys(flag, static_cast<uint32_t>(p.world), p.timeout_ns, p.status,
                            PH_RS_TILE, t);
    if (__syncthreads_and(ok ? 1 : 0) == 0) return;
    auto src = [&](int s, int v) -> const uint4* {
      const unsigned long long row = static_cast<unsigned long long>(lm) * Cfg::BM + v / VPR;
      return stage + (static_cast<unsigned long long>(s) * Ml + row) * row_vecs + n_blk * VPR +
             v % VPR;
    };
    auto dst = [&](int v, uint4 x) {
      const unsigned long long row = static_cast<unsigned long long>(lm) * Cfg::BM + v / VPR;
      out[row * row_vecs + n_blk * VPR + v % VPR] = x;
    };
    auto valid = [&](int v) -> bool {
      return static_cast<unsigned long long>(n_blk * VPR + v % VPR) < row_vecs;
    };
    switch (p.world) {
      case 1: reduce_tile_copies<1, Cfg::BM * VPR>(src, dst, valid); break;
      case 2: reduce_tile_copies<2, Cfg::BM * VPR>(src, dst, valid); break;
      case 4: reduce_tile_copies<4, Cfg::BM * VPR>(src, dst, valid); break;
      default: reduce_tile_copies<8, Cfg::BM * VPR>(src, dst, valid); break;
    }
    __syncthreads();
    if (threadIdx.x == 0) *flag = 0u;  // ready for the call after next
  }
}

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
  __syncthreads();
  rs_reduce_phase<Cfg>(p, parity, cta, ctas_per_rank);
  fused_end(p.seq, static_cast<uint32_t>(ctas_per_rank));
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
  if (emu != nullptr) {
    void* params[] = {const_cast<GemmRsParams*>(&p), &emu, &ctas_per_rank};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(gemm_rs_kernel<Cfg>),
                                    dim3(ctas_per_rank * emu_world), dim3(Cfg::THREADS), params,
                                    Cfg::SMEM_BYTES, st);
  } else {
    gemm_rs_kernel<Cfg><<<ctas_per_rank, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(p, nullptr,
                                                                              ctas_per_rank);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    set_last_error(std::string("gemm_rs launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // namespace cb

using namespace cb;

extern "C" {

struct CbGemmRsDesc {
  int rank, world;
  int M, N, K;            // K = local K shard
  int fp8;
  float alpha;
  int bn;                 // 256 or 128
  int ctas_per_rank;
  const void* a;          // [M, K]
  const void* b;          // [N, K]
  void* out;              // [M/world, N] bf16
  void* stage_peer[2][CB_MAX_RANKS];  // staging [W][M/W][N] bf16 per parity and rank
  void* flags_peer[CB_MAX_RANKS];     // uint32 [2][8192] per rank
  void* seq;
  void* status;
  unsigned long long timeout_ns;
};

static int build_rs_params(const CbGemmRsDesc& d, GemmRsParams* p) {
  const int esz = d.fp8 ? 1 : 2;
  const int BK = d.fp8 ? 128 : 64;
  const TmapDtype dt = d.fp8 ? TMAP_U8 : TMAP_BF16;
  if (d.world < 1 || d.M % (d.world * 128) != 0) {
    set_last_error("gemm_rs: M must be a multiple of world * 128");
    return -1;
  }
  if (d.K % 16 != 0 || d.N % 8 != 0) {
    set_last_error("gemm_rs: K % 16 == 0 and N % 8 == 0 required");
    return -1;
  }
  const int Ml = d.M / d.world;
  const int num_n = (d.N + d.bn - 1) / d.bn;
  if ((Ml / 128) * num_n > kRsMaxTiles) {
    set_last_error("gemm_rs: too many output tiles per rank");
    return -1;
  }
  if (make_tmap_2d(&p->tm_a, d.a, dt, d.K, d.M, (unsigned long long)d.K * esz, BK, 128, true))
    return -1;
  if (make_tmap_2d(&p->tm_b, d.b, dt, d.K, d.N, (unsigned long long)d.K * esz, BK, d.bn, true))
    return -1;
  for (int par = 0; par < 2; ++par) {
    for (int o = 0; o < CB_MAX_RANKS; ++o)
      p->stage_peer[par][o] = static_cast<uint8_t*>(d.stage_peer[par][o]);
    p->stage_local[par] = static_cast<const uint8_t*>(d.stage_peer[par][d.rank]);
  }
  p->g.M = d.M;
  p->g.N = d.N;
  p->g.K = d.K;
  p->g.num_m_blocks = d.M / 128;
  p->g.num_n_blocks = num_n;
  p->g.num_k_blocks = (d.K + BK - 1) / BK;
  p->g.alpha = d.alpha;
  p->rank = d.rank;
  p->world = d.world;
  p->blocks_per_rank = Ml / 128;
  p->raster_group = p->blocks_per_rank < 8 ? p->blocks_per_rank : 8;
  for (int r = 0; r < CB_MAX_RANKS; ++r) p->flags_peer[r] = static_cast<uint32_t*>(d.flags_peer[r]);
  p->flags_local = static_cast<uint32_t*>(d.flags_peer[d.rank]);
  p->out = d.out;
  p->seq.seq = static_cast<uint32_t*>(d.seq);
  p->seq.done_ctas = static_cast<uint32_t*>(d.seq) + 1;
  p->status = static_cast<uint32_t*>(d.status);
  p->timeout_ns = d.timeout_ns;
  return 0;
}

int cb_sizeof_gemm_rs_params() { return static_cast<int>(sizeof(GemmRsParams)); }

int cb_gemm_rs(const CbGemmRsDesc* descs, int n, void* emu_table, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n < 1 || n > CB_MAX_RANKS) return -1;
  static GemmRsParams hp[CB_MAX_RANKS];
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
    if (d.bn == 256) return launch_rs<GemmCfg<256, 4, true>>(hp[0], emu, n, d.ctas_per_rank, st);
    if (d.bn == 128) return launch_rs<GemmCfg<128, 6, true>>(hp[0], emu, n, d.ctas_per_rank, st);
  } else {
    if (d.bn == 256) return launch_rs<GemmCfg<256, 4, false>>(hp[0], emu, n, d.ctas_per_rank, st);
    if (d.bn == 128) return launch_rs<GemmCfg<128, 6, false>>(hp[0], emu, n, d.ctas_per_rank, st);
  }
  set_last_error("gemm_rs: bn must be 128 or 256");
  return -1;
}

}  // extern "C"
