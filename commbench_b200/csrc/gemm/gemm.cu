// Plain (single-GPU) tcgen05 GEMM entry points and the tensor-map helper.
// C[M,N] = alpha * A[M,K] * B[N,K]^T, bf16 or fp8-e4m3 inputs, bf16 output.
//
// This is the local GEMM every fused path is built from, and the kernel that
// runs when the world size is 1.  The reference has the equivalent as
// `matmul::kernel` (datasets/example053_thunderkitten_gemm_ar_easy/nv/
// empty_thunderkitten_gemm_ar.cu:84-191).
#include "gemm_sm100.cuh"

#include <string>

#include "../symm/driver_api.h"
#include "launch.h"
#include "tmap_host.h"

namespace cb {

int make_tmap_2d(CUtensorMap* out, const void* base, TmapDtype dt, unsigned long long inner,
                 unsigned long long outer, unsigned long long row_stride_bytes,
                 unsigned box_inner, unsigned box_outer, bool swizzle128) {
  const DriverApi& d = driver_api();
  if (!d.ok) {
    set_last_error("tensor map: " + d.why);
    return -1;
  }
  const unsigned esz = dt == TMAP_BF16 ? 2 : (dt == TMAP_U8 ? 1 : 4);
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) {
    set_last_error("tensor map: base address is not 16-byte aligned");
    return -1;
  }
  if (row_stride_bytes % 16ull != 0) {
    set_last_error("tensor map: row stride is not a multiple of 16 bytes");
    return -1;
  }
  if ((box_inner * esz) % 16u != 0 || box_inner > 256u || box_outer > 256u) {
    set_last_error("tensor map: bad box");
    return -1;
  }
  if (swizzle128 && box_inner * esz != 128u) {
    set_last_error("tensor map: 128-byte swizzle needs a 128-byte inner box");
    return -1;
  }
  const CUtensorMapDataType cdt = dt == TMAP_BF16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                  : dt == TMAP_U8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                                  : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = d.cuTensorMapEncodeTiled(
      out, cdt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuTensorMapEncodeTiled", r));
    return -1;
  }
  return 0;
}

struct PlainParams {
  CUtensorMap tm_a, tm_b, tm_c;
  GemmShape g;
  uint32_t* status;
  int raster_group;
};

template <class Cfg>
struct PlainPolicy {
  using P = PlainParams;
  static constexpr bool kDirect = false;
  static constexpr bool kSignalPerTile = false;
  static constexpr bool kScatterRows = false;
  __device__ static int b_row(const P&, int, int n_blk) { return n_blk * Cfg::BN; }
  __device__ static int num_tiles(const P& p) { return p.g.num_m_blocks * p.g.num_n_blocks; }
  __device__ static void tile_coord(const P& p, int tile, int* m, int* n) {
    raster_tile(tile, p.g.num_m_blocks, p.g.num_n_blocks, p.raster_group, m, n);
  }
  __device__ static const CUtensorMap* map_a(const P& p, int) { return &p.tm_a; }
  __device__ static const CUtensorMap* map_b(const P& p) { return &p.tm_b; }
  __device__ static int a_row(const P&, int m_blk) { return m_blk * Cfg::BM; }
  __device__ static bool wait_a_ready(const P&, int, volatile int*) { return true; }
  __device__ static void store_box(const P& p, int m_blk, int n_blk, int row, int col,
                                   const void* smem_box) {
    tma_store_2d(&p.tm_c, smem_box, n_blk * Cfg::BN + col, m_blk * Cfg::BM + row);
  }
  __device__ static void tile_done(const P&, int, int, int) {}
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
    gemm_plain_kernel(const __grid_constant__ PlainParams p) {
  extern __shared__ uint8_t smem_raw[];
  gemm_cta_main<Cfg, PlainPolicy<Cfg>>(p, p.g, p.status, blockIdx.x, gridDim.x, smem_raw);
}

static int g_sm_count = 0;
static int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_sm_count <= 0) g_sm_count = 148;
  }
  return g_sm_count;
}

template <class Cfg>
static int launch_plain(const void* a, const void* b, void* c, int M, int N, int K, float alpha,
                        uint32_t* status, int max_ctas, cudaStream_t st,
                        unsigned long long* trace = nullptr, const float* a_scale = nullptr,
                        const float* b_scale = nullptr, const uint32_t* sfa = nullptr,
                        const uint32_t* sfb = nullptr) {
  PlainParams p;
  const TmapDtype dt = Cfg::FP8 ? TMAP_U8 : TMAP_BF16;
  const unsigned esz = Cfg::FP8 ? 1 : 2;
  if (make_tmap_2d(&p.tm_a, a, dt, K, M, (unsigned long long)K * esz, Cfg::BK, Cfg::CTA_M, true))
    return -1;
  if (make_tmap_2d(&p.tm_b, b, dt, K, N, (unsigned long long)K * esz, Cfg::BK, Cfg::B_ROWS, true))
    return -1;
  if (make_tmap_2d(&p.tm_c, c, TMAP_BF16, N, M, (unsigned long long)N * 2, Cfg::EPI_COLS, 32,
                   true))
    return -1;
  p.g.M = M;
  p.g.N = N;
  p.g.K = K;
  p.g.num_m_blocks = (M + Cfg::BM - 1) / Cfg::BM;
  p.g.num_n_blocks = (N + Cfg::BN - 1) / Cfg::BN;
  p.g.num_k_blocks = (K + Cfg::BK - 1) / Cfg::BK;
  p.g.alpha = alpha;
  p.g.trace = trace;
  p.g.a_scale = a_scale;
  p.g.b_scale = b_scale;
  p.g.sfa = sfa;
  p.g.sfb = sfb;
  p.g.sfa_rows = M;
  p.g.sfb_rows = N;
  p.status = status;
  // Row blocks per raster panel: the panel's A rows (panel x K) stay in L2 while the B
  // tiles stream past them, so keep the panel near 32 MB.
  {
    const long long panel_rows = (32ll << 20) / (static_cast<long long>(K) * esz);
    int grp = static_cast<int>(panel_rows / Cfg::BM);
    if (grp < 2) grp = 2;
    if (grp > 16) grp = 16;
    p.raster_group = grp;
  }
  {
    cudaError_t e = cudaFuncSetAttribute(gemm_plain_kernel<Cfg>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM_BYTES);
    if (e != cudaSuccess) {
      set_last_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
      return -1;
    }
  }
  int tiles = p.g.num_m_blocks * p.g.num_n_blocks;
  int ctas = sm_count();
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  if (tiles * Cfg::PAIR < ctas) ctas = tiles * Cfg::PAIR;
  ctas -= ctas % Cfg::PAIR;
  if (ctas < Cfg::PAIR) return 0;
  cudaError_t e = launch_gemm_kernel(gemm_plain_kernel<Cfg>, ctas, Cfg::THREADS, Cfg::SMEM_BYTES,
                                     st, Cfg::PAIR, false, p);
  if (e != cudaSuccess) {
    set_last_error(std::string("gemm launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // namespace cb

using namespace cb;

extern "C" {

// bf16: A [M,K], B [N,K], C [M,N], all row-major and 16-byte aligned; K % 8 == 0, N % 8 == 0.
// `bn` picks the tile: 256, 128 or 64 = one CTA per 128 x bn tile; 512 = a CTA pair per
// 256 x 256 tile, 384 = a pair per 256 x 128 tile; 0 = choose from the shape.
// `status` may be null.  Returns 0 or -1 (cb_last_error()).
int cb_gemm_bf16(const void* a, const void* b, void* c, int M, int N, int K, float alpha, int bn,
                 int max_ctas, void* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 8) != 0 || (N % 8) != 0) {
    set_last_error("cb_gemm_bf16: need M,N,K > 0, K % 8 == 0, N % 8 == 0");
    return -1;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* s = static_cast<uint32_t*>(status);
  if (bn == 0) {
    // Fill the machine: pairs on 256 x 256 tiles when there are plenty of them, narrower
    // tiles for skinny problems.
    const long long m_blocks = (M + 127) / 128;
    if (((M + 255) / 256) * ((N + 255) / 256) * 2 >= sm_count()) bn = 512;
    else if (m_blocks * ((N + 255) / 256) >= sm_count()) bn = 256;
    else if (m_blocks * ((N + 127) / 128) >= sm_count()) bn = 128;
    else bn = 64;
  }
  switch (bn) {
    case 512:
      return launch_plain<GemmCfg<256, 6, false, 2>>(a, b, c, M, N, K, alpha, s, max_ctas, st);
    case 384:
      return launch_plain<GemmCfg<128, 8, false, 2>>(a, b, c, M, N, K, alpha, s, max_ctas, st);
    case 256:
      return launch_plain<GemmCfg<256, 4, false>>(a, b, c, M, N, K, alpha, s, max_ctas, st);
    case 128:
      return launch_plain<GemmCfg<128, 6, false>>(a, b, c, M, N, K, alpha, s, max_ctas, st);
    case 64:
      return launch_plain<GemmCfg<64, 8, false>>(a, b, c, M, N, K, alpha, s, max_ctas, st);
    default:
      set_last_error("cb_gemm_bf16: bn must be 0, 64, 128, 256, 384 or 512");
      return -1;
  }
}

// cb_gemm_bf16 with the role trace switched on: `trace` = 8 x (number of SMs) 64-bit words
// of device memory (see GemmShape::trace for what each CTA writes).  bn: 512 or 256.
int cb_gemm_bf16_traced(const void* a, const void* b, void* c, int M, int N, int K, float alpha,
                        int bn, void* trace, void* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 8) != 0 || (N % 8) != 0 || trace == nullptr) {
    set_last_error("cb_gemm_bf16_traced: need M,N,K > 0, K % 8 == 0, N % 8 == 0, a trace buffer");
    return -1;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* s = static_cast<uint32_t*>(status);
  unsigned long long* t = static_cast<unsigned long long*>(trace);
  if (bn == 512)
    return launch_plain<GemmCfg<256, 6, false, 2>>(a, b, c, M, N, K, alpha, s, 0, st, t);
  if (bn == 256) return launch_plain<GemmCfg<256, 4, false>>(a, b, c, M, N, K, alpha, s, 0, st, t);
  set_last_error("cb_gemm_bf16_traced: bn must be 256 or 512");
  return -1;
}

// fp8 e4m3 inputs with ONE scale per tensor folded into alpha; K % 16 == 0.
int cb_gemm_fp8(const void* a, const void* b, void* c, int M, int N, int K, float alpha, int bn,
                int max_ctas, void* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 16) != 0 || (N % 8) != 0) {
    set_last_error("cb_gemm_fp8: need M,N,K > 0, K % 16 == 0, N % 8 == 0");
    return -1;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* s = static_cast<uint32_t*>(status);
  if (bn == 0) {
    const long long m_blocks = (M + 127) / 128;
    if (((M + 255) / 256) * ((N + 255) / 256) * 2 >= sm_count()) bn = 512;
    else if (m_blocks * ((N + 255) / 256) >= sm_count()) bn = 256;
    else if (m_blocks * ((N + 127) / 128) >= sm_count()) bn = 128;
    else bn = 64;
  }
  switch (bn) {
    case 512:
      return launch_plain<GemmCfg<256, 6, true, 2>>(a, b, c, M, N, K, alpha, s, max_ctas, st);
    case 256:
      return launch_plain<GemmCfg<256, 4, true>>(a, b, c, M, N, K, alpha, s, max_ctas, st);
    case 128:
      return launch_plain<GemmCfg<128, 6, true>>(a, b, c, M, N, K, alpha, s, max_ctas, st);
    case 64:
      return launch_plain<GemmCfg<64, 8, true>>(a, b, c, M, N, K, alpha, s, max_ctas, st);
    default:
      set_last_error("cb_gemm_fp8: bn must be 0, 64, 128, 256 or 512");
      return -1;
  }
}

// Block-scaled fp8: a [M,K] e4m3 with a_scale [M, K/128] fp32 (one scale per row and 128
// columns), b [N,K] e4m3 with b_scale [ceil(N/128), K/128] (one per 128 x 128 block); K % 128 == 0.
// C = alpha * (a * a_scale) (b * b_scale)^T in bf16.  The quantised operands feed the tensor
// cores directly; every 128-wide K block's partial sum is scaled and accumulated in fp32
// registers.  pair != 0: CTA pairs (256 x 256 tiles), else one CTA per 128 x 256 tile.
int cb_gemm_fp8_blockscaled(const void* a, const void* a_scale, const void* b, const void* b_scale,
                            void* c, int M, int N, int K, float alpha, int pair, int max_ctas,
                            void* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 128) != 0 || (N % 8) != 0 || a_scale == nullptr ||
      b_scale == nullptr) {
    set_last_error("cb_gemm_fp8_blockscaled: need M,N,K > 0, K % 128 == 0, N % 8 == 0, scales");
    return -1;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* s = static_cast<uint32_t*>(status);
  const float* as = static_cast<const float*>(a_scale);
  const float* bs = static_cast<const float*>(b_scale);
  if (pair)
    return launch_plain<GemmCfg<256, 5, true, 2, true>>(a, b, c, M, N, K, alpha, s, max_ctas, st,
                                                        nullptr, as, bs);
  return launch_plain<GemmCfg<256, 3, true, 1, true>>(a, b, c, M, N, K, alpha, s, max_ctas, st,
                                                      nullptr, as, bs);
}

// Block-scaled fp8 with POWER-OF-TWO scales applied by the tensor core: a [M,K], b [N,K] e4m3;
// sfa [ceil(K/512), M] and sfb [ceil(K/512), N] 32-bit words, each packing the exponent bytes
// (value 2^(byte - 127)) of four consecutive 128-wide K blocks of one operand row, lowest byte
// first (cb_quant_blockscaled_pow2 writes them; for a 128 x 128-block weight every row of a
// block carries the block's byte).  K % 128 == 0.
int cb_gemm_fp8_mx_traced(const void* a, const void* sfa, const void* b, const void* sfb, void* c,
                          int M, int N, int K, float alpha, int max_ctas, void* trace,
                          void* status, void* stream);

int cb_gemm_fp8_mx(const void* a, const void* sfa, const void* b, const void* sfb, void* c, int M,
                   int N, int K, float alpha, int max_ctas, void* status, void* stream) {
  return cb_gemm_fp8_mx_traced(a, sfa, b, sfb, c, M, N, K, alpha, max_ctas, nullptr, status,
                               stream);
}

// The same with the MMA role's trace on (`trace`: 8 x number-of-SMs 64-bit words, may be null).
int cb_gemm_fp8_mx_traced(const void* a, const void* sfa, const void* b, const void* sfb, void* c,
                          int M, int N, int K, float alpha, int max_ctas, void* trace,
                          void* status, void* stream) {
  // max_ctas < 0 selects the one-CTA-per-tile form (128 x 192 tiles) instead of CTA pairs.
  const bool single = max_ctas < 0;
  if (single) max_ctas = 0;
  if (M <= 0 || N <= 0 || K <= 0 || (K % 128) != 0 || (N % 8) != 0 || sfa == nullptr ||
      sfb == nullptr) {
    set_last_error("cb_gemm_fp8_mx: need K % 128 == 0, N % 8 == 0 and both scale arrays");
    return -1;
  }
  if (single)
    return launch_plain<GemmCfg<192, 4, true, 1, false, true>>(
        a, b, c, M, N, K, alpha, static_cast<uint32_t*>(status), max_ctas,
        static_cast<cudaStream_t>(stream), static_cast<unsigned long long*>(trace), nullptr,
        nullptr, static_cast<const uint32_t*>(sfa), static_cast<const uint32_t*>(sfb));
  return launch_plain<GemmCfg<192, 6, true, 2, false, true>>(
      a, b, c, M, N, K, alpha, static_cast<uint32_t*>(status), max_ctas,
      static_cast<cudaStream_t>(stream), static_cast<unsigned long long*>(trace), nullptr, nullptr,
      static_cast<const uint32_t*>(sfa), static_cast<const uint32_t*>(sfb));
}

}  // extern "C"
