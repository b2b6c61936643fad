// Block-scaled fp8 (e4m3) operands: activations carry one fp32 scale per 1 x 128 block
// along K, weights one per 128 x 128 block.  These kernels expand them to bf16 so that the
// bf16 tcgen05 GEMMs (plain and fused) consume them: fp8 halves the bytes that are stored and
// moved, the tensor cores run in bf16.  (The reference's fp8 GEMMs are unscaled:
// datasets/example052_thunderkitten_ag_gemm_fp8_easy/nv/empty_thunderkitten_ag_gemm_fp8.cu:92-122.)
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace cb {
void set_last_error(const std::string& s);

// x [rows, K] e4m3; scale [rows / rb, K / 128] with rb = 1 (activations) or 128 (weights).
__global__ void dequant_blockscaled_kernel(const uint8_t* __restrict__ x,
                                           const float* __restrict__ scale,
                                           __nv_bfloat16* __restrict__ out, long long rows, int K,
                                           int rb) {
  const long long vec_per_row = K / 8;
  const long long total = rows * vec_per_row;
  const int kblocks = K / 128;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / vec_per_row;
    const int v = static_cast<int>(idx % vec_per_row);
    const float s = scale[(r / rb) * kblocks + v / 16];
    const uint2 raw = *reinterpret_cast<const uint2*>(x + r * K + v * 8);
    const __nv_fp8x2_storage_t* p8 = reinterpret_cast<const __nv_fp8x2_storage_t*>(&raw);
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(p8[i], __NV_E4M3);
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
      ob[i] = __floats2bfloat162_rn(f.x * s, f.y * s);
    }
    *reinterpret_cast<uint4*>(out + r * K + v * 8) = o;
  }
}

// bf16 [rows, K] -> e4m3 + scales (rb = 1: one scale per row and 128 columns; rb = 128: one
// per 128 x 128 block).  One warp per (row block, k block).
//
// pow2 != 0: the scale is rounded UP to a power of two (so that it is exactly representable as an
// 8-bit exponent, "UE8M0", the scale format the tensor cores apply in hardware) and, when
// `sf_bytes` is given, its exponent byte is also written there in the packed layout of the
// block-scaled GEMM: byte (kb % 4) of the 32-bit word [kb / 4][row], `sf_ld` = rows per K group.
// For rb = 128 the byte is replicated to every row of the block (one byte per output column
// of a GEMM and K block).
__global__ void quant_blockscaled_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                         float* __restrict__ scale, long long rows, int K, int rb,
                                         int pow2, uint8_t* __restrict__ sf_bytes, int sf_ld) {
  const int kblocks = K / 128;
  const long long nblocks = ((rows + rb - 1) / rb) * kblocks;
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= nblocks) return;
  const long long br = w / kblocks;
  const int kb = static_cast<int>(w % kblocks);
  const long long r0 = br * rb;
  const long long r1 = r0 + rb < rows ? r0 + rb : rows;
  float amax = 0.f;
  for (long long r = r0; r < r1; ++r) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(x + r * K + kb * 128 + lane * 4);
    const __nv_bfloat162 h2 =
        *reinterpret_cast<const __nv_bfloat162*>(x + r * K + kb * 128 + lane * 4 + 2);
    const float2 a = __bfloat1622float2(h), b = __bfloat1622float2(h2);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
  }
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  float s = amax > 0.f ? amax / 448.f : 1.f;
  if (pow2) {
    // smallest power of two >= s (clamped to the normal range): bump the exponent when any
    // mantissa bit is set
    uint32_t bits = __float_as_uint(s);
    uint32_t e = (bits >> 23) & 0xffu;
    if ((bits & 0x7fffffu) != 0u) ++e;
    if (e < 1u) e = 1u;
    if (e > 254u) e = 254u;
    s = __uint_as_float(e << 23);
    if (sf_bytes != nullptr)
      for (long long r = r0 + lane; r < r1; r += 32)
        sf_bytes[(static_cast<long long>(kb >> 2) * sf_ld + r) * 4 + (kb & 3)] =
            static_cast<uint8_t>(e);
  }
  const float inv = 1.f / s;
  if (lane == 0) scale[br * kblocks + kb] = s;
  for (long long r = r0; r < r1; ++r) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(x + r * K + kb * 128 + lane * 4);
    const __nv_bfloat162 h2 =
        *reinterpret_cast<const __nv_bfloat162*>(x + r * K + kb * 128 + lane * 4 + 2);
    const float2 a = __bfloat1622float2(h), b = __bfloat1622float2(h2);
    const __nv_fp8x2_storage_t lo =
        __nv_cvt_float2_to_fp8x2(make_float2(a.x * inv, a.y * inv), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi =
        __nv_cvt_float2_to_fp8x2(make_float2(b.x * inv, b.y * inv), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(q + r * K + kb * 128 + lane * 4) =
        static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
  }
}

}  // namespace cb

using namespace cb;

extern "C" {

int cb_dequant_blockscaled(const void* x, const void* scale, void* out, long long rows, int K,
                           int row_block, void* stream) {
  if (K % 128 != 0 || (row_block != 1 && row_block != 128)) {
    set_last_error("block scales: K must be a multiple of 128 and row_block 1 or 128");
    return -1;
  }
  dequant_blockscaled_kernel<<<1184, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(x), static_cast<const float*>(scale),
      static_cast<__nv_bfloat16*>(out), rows, K, row_block);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int cb_quant_blockscaled(const void* x, void* q, void* scale, long long rows, int K, int row_block,
                         void* stream) {
  if (K % 128 != 0 || (row_block != 1 && row_block != 128)) {
    set_last_error("block scales: K must be a multiple of 128 and row_block 1 or 128");
    return -1;
  }
  const long long nblocks = ((rows + row_block - 1) / row_block) * (K / 128);
  const int threads = 256;
  const long long blocks = (nblocks * 32 + threads - 1) / threads;
  quant_blockscaled_kernel<<<static_cast<unsigned>(blocks), threads, 0,
                             static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), static_cast<float*>(scale),
      rows, K, row_block, 0, nullptr, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Same with power-of-two scales; `sf_words` = ceil(K / 512) x sf_rows 32-bit words (sf_rows >=
// rows; pre-filled with 0x7f7f7f7f = 1.0 by the caller) receives the packed exponent bytes (see
// the kernel).  Feeds cb_gemm_fp8_mx.
int cb_quant_blockscaled_pow2(const void* x, void* q, void* scale, void* sf_words, int sf_rows,
                              long long rows, int K, int row_block, void* stream) {
  const void* sf_bytes = sf_words;
  const int sf_ld = sf_rows;
  if (K % 128 != 0 || (row_block != 1 && row_block != 128) || sf_rows < rows) {
    set_last_error("block scales: K % 128 == 0, row_block 1 or 128, sf_rows >= rows");
    return -1;
  }
  const long long nblocks = ((rows + row_block - 1) / row_block) * (K / 128);
  const int threads = 256;
  const long long blocks = (nblocks * 32 + threads - 1) / threads;
  quant_blockscaled_kernel<<<static_cast<unsigned>(blocks), threads, 0,
                             static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), static_cast<float*>(scale),
      rows, K, row_block, 1, static_cast<uint8_t*>(const_cast<void*>(sf_bytes)), sf_ld);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
