// Fused GEMM -> all-reduce:
//   out[M, N] (on every rank) = sum over ranks q of  A_q[M, K_local] * B_q[N, K_local]^T
//
// ONE kernel per rank, two variants chosen by the host from the row count:
//  * two-shot (default): output tile t is owned by rank t % W.  The GEMM
//    epilogue writes each bf16 partial tile into the owner's staging slot
//    and bumps an arrival counter there; the owner adds the W partials in fp32
//    and writes the reduced tile into EVERY rank's symmetric result buffer (one
//    multimem.st per vector when a multicast object is bound, W plain stores
//    otherwise), then bumps each rank's "tiles done" counter; the kernel ends
//    when all tiles are done, and the result stays in the symmetric buffer.
//  * one-shot (decode-sized M): every rank sends its partial tile to ALL ranks
//    and each rank reduces every tile locally - one NVLink hop instead of two.
//
// The reference runs GEMM, barrier, multimem all-reduce, barrier as separate
// launches (datasets/example053_thunderkitten_gemm_ar_easy/nv/
// empty_thunderkitten_gemm_ar.cu:200-238 and :528-536); here the reduction
// starts as soon as the first tile leaves the tensor cores.
#include "fused_common.cuh"

#include <string>

#include "../gemm/tmap_host.h"
#include "../symm/driver_api.h"

namespace cb {

static constexpr int kArMaxTiles = 8192;  // flags per parity

struct GemmArParams {
  CUtensorMap tm_a;
  CUtensorMap tm_b;
  uint8_t* stage_peer[2][CB_MAX_RANKS];  // [parity][dest]: dest's staging [W][slots][128][BN]
  GemmShape g;
  int rank, world;
  int oneshot;
  int slots;            // staging tile slots per source on each rank
  int raster_group;
  const uint8_t* stage_local[2];          // [W][slots][128][BN] bf16
  uint32_t* flags_peer[CB_MAX_RANKS];     // [2][kArMaxTiles] arrival counters + [2] done counters
  uint32_t* flags_local;
  uint8_t* result_peer[2][CB_MAX_RANKS];  // symmetric result [M][N] bf16 (two-shot)
  uint8_t* result_mc[2];
  void* out;                              // local output or nullptr (result stays symmetric)
  FusedSeq seq;
  uint32_t* status;
  unsigned long long timeout_ns;
  unsigned long long* trace;  // optional [ctas][8] %globaltimer stamps per CTA (nullptr: off)
  int poll_ns;                // sleep between polls of a flag
};

// Optional tracing: thread 0 of each CTA stamps %globaltimer at the kernel's phase changes.
__device__ __forceinline__ void ar_stamp(const GemmArParams& p, int cta, int slot) {
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[cta * 8 + slot] = globaltimer_ns();
}

__device__ __forceinline__ bool ar_wait(const GemmArParams& p, const uint32_t* flag, uint32_t target,
                                        uint32_t phase, uint32_t detail) {
  return wait_flag_ge_sys_paced(flag, target, p.timeout_ns, p.status, phase, detail,
                                static_cast<uint32_t>(p.poll_ns));
}

// done counters sit after the arrival counters of both parities
__device__ __host__ constexpr int ar_done_index(int parity) { return 2 * kArMaxTiles + parity; }

struct ArRt {
  const GemmArParams* p;
  uint32_t parity;
};

template <class Cfg>
struct ArPolicy {
  __device__ static int num_tiles(const ArRt& r) {
    return r.p->g.num_m_blocks * r.p->g.num_n_blocks;
  }
  __device__ static void tile_coord(const ArRt& r, int tile, int* m, int* n) {
    // Rotate the start by rank so the ranks' early tiles go to different owners.
    const int nt = num_tiles(r);
    int t = tile + (nt / r.p->world) * r.p->rank;
    if (t >= nt) t -= nt;
    *m = t / r.p->g.num_n_blocks;
    *n = t - *m * r.p->g.num_n_blocks;
  }
  __device__ static const CUtensorMap* map_a(const ArRt& r, int) { return &r.p->tm_a; }
  __device__ static const CUtensorMap* map_b(const ArRt& r) { return &r.p->tm_b; }
  __device__ static int a_row(const ArRt&, int m_blk) { return m_blk * Cfg::BM; }
  __device__ static bool wait_a_ready(const ArRt&, int, volatile int*) { return true; }
  static constexpr bool kDirect = true;
  static constexpr bool kSignalPerTile = true;
  static constexpr bool kScatterRows = false;
  __device__ static int b_row(const ArRt&, int, int n_blk) { return n_blk * Cfg::BN; }
  __device__ static void direct_targets(const ArRt& r, int m_blk, int n_blk, DirectTargets* t) {
    const GemmArParams& p = *r.p;
    const int tl = m_blk * p.g.num_n_blocks + n_blk;
    const long long tile_bytes = static_cast<long long>(Cfg::BM) * Cfg::BN * 2;
    t->ld_bytes = static_cast<long long>(Cfg::BN) * 2;
    const int rows_left = p.g.M - m_blk * Cfg::BM;
    t->rows = rows_left < Cfg::BM ? rows_left : Cfg::BM;  // rows past M carry nothing
    t->cols = Cfg::BN;
    if (p.oneshot) {
      t->n = p.world;
      for (int d = 0; d < p.world; ++d) {
        const int dest = (p.rank + d) % p.world;
        t->base[d] = p.stage_peer[r.parity][dest] +
                     (static_cast<long long>(p.rank) * p.slots + tl) * tile_bytes;
      }
    } else {
      t->n = 1;
      t->base[0] = p.stage_peer[r.parity][tl % p.world] +
                   (static_cast<long long>(p.rank) * p.slots + tl / p.world) * tile_bytes;
    }
  }
  __device__ static void tile_done(const ArRt& r, int m_blk, int n_blk, int) {
    const GemmArParams& p = *r.p;
    const int t = m_blk * p.g.num_n_blocks + n_blk;
    if (p.oneshot) {
      for (int d = 0; d < p.world; ++d) {
        const int dest = (p.rank + d) % p.world;
        red_relaxed_sys_add(p.flags_peer[dest] + r.parity * kArMaxTiles + t, 1u);
      }
    } else {
      red_relaxed_sys_add(p.flags_peer[t % p.world] + r.parity * kArMaxTiles + t / p.world, 1u);
    }
  }
};

template <class Cfg>
__device__ __forceinline__ void ar_reduce_phase(const GemmArParams& p, uint32_t call, int cta,
                                                int num_ctas) {
  const uint32_t parity = call & 1u;
  const int ntiles = p.g.num_m_blocks * p.g.num_n_blocks;
  constexpr int VPR = Cfg::BN / 8;
  constexpr int TILE_VECS = Cfg::BM * VPR;
  const uint4* stage = reinterpret_cast<const uint4*>(p.stage_local[parity]);
  const unsigned long long row_vecs = static_cast<unsigned long long>(p.g.N) / 8ull;
  // Tiles this rank reduces: all of them (one-shot) or the ones it owns (two-shot).
  const int my_tiles = p.oneshot ? ntiles : (ntiles - p.rank + p.world - 1) / p.world;
  for (int i = cta; i < my_tiles; i += num_ctas) {
    const int slot = i;
    const int t = p.oneshot ? i : i * p.world + p.rank;
    const int m_blk = t / p.g.num_n_blocks;
    const int n_blk = t - m_blk * p.g.num_n_blocks;
    uint32_t* flag = p.flags_local + parity * kArMaxTiles + slot;
    bool ok = true;
    if (threadIdx.x == 0)
      ok = ar_wait(p, flag, static_cast<uint32_t>(p.world), PH_AR_TILE, t);
    if (__syncthreads_and(ok ? 1 : 0) == 0) return;
    if (i == cta) ar_stamp(p, cta, 5);
    auto src = [&](int s, int v) -> const uint4* {
      return stage + (static_cast<unsigned long long>(s) * p.slots + slot) * TILE_VECS + v;
    };
    auto valid = [&](int v) -> bool {
      return m_blk * Cfg::BM + v / VPR < p.g.M &&
             static_cast<unsigned long long>(n_blk * VPR + v % VPR) < row_vecs;
    };
    auto dst = [&](int v, uint4 sum) {
      const unsigned long long o =
          static_cast<unsigned long long>(m_blk * Cfg::BM + v / VPR) * row_vecs + n_blk * VPR +
          v % VPR;
      if (p.oneshot) {
        static_cast<uint4*>(p.out)[o] = sum;
      } else if (p.result_mc[parity] != nullptr) {
        mm_st_v4(reinterpret_cast<uint4*>(p.result_mc[parity]) + o, sum);
      } else {
        for (int d = 0; d < p.world; ++d) {
          const int dest = (p.rank + d) % p.world;
          st_sys_v4(reinterpret_cast<uint4*>(p.result_peer[parity][dest]) + o, sum);
        }
      }
    };
    switch (p.world) {
      case 1: reduce_tile_copies<1, TILE_VECS>(src, dst, valid); break;
      case 2: reduce_tile_copies<2, TILE_VECS>(src, dst, valid); break;
      case 4: reduce_tile_copies<4, TILE_VECS>(src, dst, valid); break;
      default: reduce_tile_copies<8, TILE_VECS>(src, dst, valid); break;
    }
    __syncthreads();
    if (i == cta) ar_stamp(p, cta, 6);
    if (threadIdx.x == 0) {
      *flag = 0u;
      if (!p.oneshot) {
        fence_acq_rel_sys();  // release for the whole CTA's stores (ordered by the barrier)
        if (i == cta) ar_stamp(p, cta, 7);
        for (int d = 0; d < p.world; ++d) {
          const int dest = (p.rank + d) % p.world;
          red_relaxed_sys_add(p.flags_peer[dest] + ar_done_index(parity), 1u);
        }
      }
    }
  }
  ar_stamp(p, cta, 2);
  if (p.oneshot) return;
  // Two-shot: the kernel must not end before every owner has delivered its reduced tiles
  // into this rank's result buffer.  ONE thread of the grid waits for that (CTA 0, polling
  // at a modest rate); the other CTAs leave, and the end of the kernel is what publishes
  // the result to the stream.  Letting every CTA poll - the remote counter or a local copy
  // of it - slowed the peers' traffic into this GPU by hundreds of microseconds.
  if (cta != 0) return;
  uint32_t* done = p.flags_local + ar_done_index(parity);
  bool ok = true;
  if (threadIdx.x == 0) ok = ar_wait(p, done, static_cast<uint32_t>(ntiles), PH_AR_DONE, 0);
  if (__syncthreads_and(ok ? 1 : 0) == 0) return;
  ar_stamp(p, cta, 3);
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
    gemm_ar_kernel(const __grid_constant__ GemmArParams p0, const GemmArParams* emu,
                   int ctas_per_rank) {
  extern __shared__ uint8_t smem_raw[];
  const int vrank = emu != nullptr ? blockIdx.x / ctas_per_rank : 0;
  const GemmArParams& p = emu != nullptr ? emu[vrank] : p0;
  const int cta = blockIdx.x - vrank * ctas_per_rank;
  const uint32_t call = ld_volatile(p.seq.seq);  // every thread reads it before anyone bumps it
  const uint32_t parity = call & 1u;
  ar_stamp(p, cta, 0);
  ArRt rt{&p, parity};
  gemm_cta_main<Cfg, ArPolicy<Cfg>>(rt, p.g, p.status, cta, ctas_per_rank, smem_raw);
  __syncthreads();
  ar_stamp(p, cta, 1);
  ar_reduce_phase<Cfg>(p, call, cta, ctas_per_rank);
  ar_stamp(p, cta, 4);
  // Last CTA out clears this parity's done counter (every CTA has seen it complete).
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(p.seq.done_ctas, 1u);
    if (prev == static_cast<uint32_t>(ctas_per_rank) - 1u) {
      p.flags_local[ar_done_index(parity)] = 0u;
      *p.seq.done_ctas = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.seq.seq) = ld_volatile(p.seq.seq) + 1u;
    }
  }
}

template <class Cfg>
static int launch_ar(const GemmArParams& p, const GemmArParams* emu, int emu_world,
                     int ctas_per_rank, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(gemm_ar_kernel<Cfg>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    return -1;
  }
  if (emu != nullptr) {
    void* params[] = {const_cast<GemmArParams*>(&p), &emu, &ctas_per_rank};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(gemm_ar_kernel<Cfg>),
                                    dim3(ctas_per_rank * emu_world), dim3(Cfg::THREADS), params,
                                    Cfg::SMEM_BYTES, st);
  } else {
    gemm_ar_kernel<Cfg><<<ctas_per_rank, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(p, nullptr,
                                                                              ctas_per_rank);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    set_last_error(std::string("gemm_ar launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // namespace cb

using namespace cb;

extern "C" {

struct CbGemmArDesc {
  int rank, world;
  int M, N, K;
  int fp8;
  float alpha;
  int bn;         // 64, 128 or 256
  int oneshot;
  int slots;      // staging tile slots per source rank (>= tiles reduced by one rank)
  int ctas_per_rank;
  const void* a;  // [M, K]
  const void* b;  // [N, K]
  void* out;      // one-shot: [M, N] bf16 local.  two-shot: nullptr (result_peer[parity][rank])
  void* stage_peer[2][CB_MAX_RANKS];   // [W][slots][128][bn] bf16
  void* result_peer[2][CB_MAX_RANKS];  // [M][N] bf16 (two-shot only)
  void* result_mc[2];
  void* flags_peer[CB_MAX_RANKS];      // uint32 [2*8192 + 2]
  void* seq;
  void* status;
  unsigned long long timeout_ns;
  void* trace;  // optional uint64 [ctas_per_rank][8]: per-CTA phase time stamps, or nullptr
  int poll_ns;  // sleep between flag polls in nanoseconds
};

static int build_ar_params(const CbGemmArDesc& d, GemmArParams* p) {
  const int esz = d.fp8 ? 1 : 2;
  const int BK = d.fp8 ? 128 : 64;
  const TmapDtype dt = d.fp8 ? TMAP_U8 : TMAP_BF16;
  if (d.K % 16 != 0 || d.N % 8 != 0 || d.M < 1) {
    set_last_error("gemm_ar: K % 16 == 0, N % 8 == 0, M >= 1 required");
    return -1;
  }
  const int num_m = (d.M + 127) / 128;
  const int num_n = (d.N + d.bn - 1) / d.bn;
  const int ntiles = num_m * num_n;
  const int need_slots = d.oneshot ? ntiles : (ntiles + d.world - 1) / d.world;
  if (need_slots > d.slots || need_slots > kArMaxTiles) {
    set_last_error("gemm_ar: not enough staging slots");
    return -1;
  }
  if (d.oneshot && d.out == nullptr) {
    set_last_error("gemm_ar: the one-shot variant needs a local output");
    return -1;
  }
  if (!d.oneshot && d.out != nullptr) {
    set_last_error("gemm_ar: the two-shot variant leaves its result in result_peer[parity][rank]");
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
    for (int r = 0; r < CB_MAX_RANKS; ++r)
      p->result_peer[par][r] = static_cast<uint8_t*>(d.result_peer[par][r]);
    p->result_mc[par] = static_cast<uint8_t*>(d.result_mc[par]);
  }
  p->g.M = d.M;
  p->g.N = d.N;
  p->g.K = d.K;
  p->g.num_m_blocks = num_m;
  p->g.num_n_blocks = num_n;
  p->g.num_k_blocks = (d.K + BK - 1) / BK;
  p->g.alpha = d.alpha;
  p->rank = d.rank;
  p->world = d.world;
  p->oneshot = d.oneshot;
  p->slots = d.slots;
  p->raster_group = 8;
  for (int r = 0; r < CB_MAX_RANKS; ++r) p->flags_peer[r] = static_cast<uint32_t*>(d.flags_peer[r]);
  p->flags_local = static_cast<uint32_t*>(d.flags_peer[d.rank]);
  p->out = d.out;
  p->seq.seq = static_cast<uint32_t*>(d.seq);
  p->seq.done_ctas = static_cast<uint32_t*>(d.seq) + 1;
  p->status = static_cast<uint32_t*>(d.status);
  p->timeout_ns = d.timeout_ns;
  p->trace = static_cast<unsigned long long*>(d.trace);
  p->poll_ns = d.poll_ns;
  return 0;
}

int cb_sizeof_gemm_ar_params() { return static_cast<int>(sizeof(GemmArParams)); }
int cb_gemm_ar_flag_words() { return 2 * kArMaxTiles + 2; }

int cb_gemm_ar(const CbGemmArDesc* descs, int n, void* emu_table, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n < 1 || n > CB_MAX_RANKS) return -1;
  static GemmArParams hp[CB_MAX_RANKS];
  for (int i = 0; i < n; ++i)
    if (build_ar_params(descs[i], &hp[i]) != 0) return -1;
  const GemmArParams* emu = nullptr;
  if (n > 1) {
    if (emu_table == nullptr) {
      set_last_error("gemm_ar: emulation needs a device table");
      return -1;
    }
    cudaError_t e = cudaMemcpyAsync(emu_table, hp, sizeof(GemmArParams) * n,
                                    cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) {
      set_last_error(std::string("gemm_ar: table copy: ") + cudaGetErrorString(e));
      return -1;
    }
    cudaStreamSynchronize(st);
    emu = static_cast<const GemmArParams*>(emu_table);
  }
  const CbGemmArDesc& d = descs[0];
#define CB_AR_CASE(BN, ST)                                                                     \
  if (d.bn == BN) {                                                                            \
    return d.fp8 ? launch_ar<GemmCfg<BN, ST, true>>(hp[0], emu, n, d.ctas_per_rank, st)        \
                 : launch_ar<GemmCfg<BN, ST, false>>(hp[0], emu, n, d.ctas_per_rank, st);      \
  }
  CB_AR_CASE(256, 4)
  CB_AR_CASE(128, 6)
  CB_AR_CASE(64, 8)
#undef CB_AR_CASE
  set_last_error("gemm_ar: bn must be 64, 128 or 256");
  return -1;
}

}  // extern "C"
