// Flash-attention forward on tcgen05 (bf16, head_dim 128, causal or full, GQA),
// producing the normalised output of ONE key/value chunk plus the row-wise
// log-sum-exp, so that chunks (ring steps, context-parallel shards) can be merged
// exactly afterwards with `attn_merge`.
//
// The reference's context-parallel examples move K/V (ring) or Q/K/V/O (Ulysses)
// and leave the attention math out (datasets/example069_thunderkitten_ring_attn_hard/nv/
// empty_thunderkitten_ring_attn.cu:11-19, datasets/example070_thunderkitten_ulysses_attn_hard/nv/
// empty_thunderkitten_ulysses_attn.cu:11-25); this file supplies it.
//
// One CTA per (128 query rows, query head, batch):
//   warp 0     TMA producer: Q once, then K and V tiles of 128 keys, two stages
//   warp 1     MMA issuer:   S = Q K^T   (M=128, N=128 keys, K=128 over head_dim)
//                            PV = P V    (M=128, N=128 head_dim, K=128 over keys; V is the
//                                         MN-major operand, read in place as TMA wrote it)
//   warps 2-5  softmax: one query row per thread; S comes out of TMEM in 32-column
//              chunks (two passes: row max, then exp/sum), P goes to shared memory in the
//              swizzled K-major layout the second MMA reads, O lives in registers
//              (O = O * alpha + PV after each block).
// S, P and PV are double-buffered so QK^T of block j+1 and P*V of block j-1 both overlap the
// softmax of block j.
// Every mbarrier wait is bounded (see mbarrier.cuh).
#include <cuda.h>
#include <cuda_bf16.h>

#include <string>

#include "../gemm/tmap_host.h"
#include "../prim/tcgen05.cuh"
#include "../prim/tma.cuh"
#include "../symm/driver_api.h"

namespace cb {

static constexpr int FA_BM = 128;   // query rows per CTA
static constexpr int FA_BN = 128;   // keys per block
static constexpr int FA_D = 128;    // head dim
static constexpr int FA_SUB = 16384;  // bytes of one [128 x 64] bf16 sub-tile
static constexpr int FA_SMEM = 2 * FA_SUB /*Q*/ + 2 * 2 * FA_SUB /*K x2*/ + 2 * 2 * FA_SUB /*V x2*/ +
                               2 * 2 * FA_SUB /*P x2*/ + 1024;
static constexpr int FA_THREADS = 192;

struct FaParams {
  CUtensorMap tm_q;  // 3-D {D, Hq, B*Sq}, box {64, 1, 128}
  CUtensorMap tm_k;  // 3-D {D, Hkv, B*Skv}
  CUtensorMap tm_v;
  __nv_bfloat16* o;  // [B, Sq, Hq, D]
  float* lse;        // [B, Hq, Sq]  (natural log; -inf for rows that saw no key)
  int B, Sq, Skv, Hq, Hkv;
  int q_offset, kv_offset;  // global sequence positions of row 0 / key 0 (causal mask)
  int causal;
  float scale_log2;         // softmax scale * log2(e)
  uint32_t* status;
};

struct FaCtl {
  uint64_t q_full;
  uint64_t k_full[2], v_full[2], kv_empty[2];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full[2], p_empty[2];
  uint64_t pv_full[2], pv_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// MN-major B operand (V as stored: [keys][d], d contiguous, 128-byte swizzle):
// leading-byte-offset = distance between the two 64-wide d sub-tiles, stride-byte-offset
// = distance between groups of 8 keys.
__device__ __forceinline__ uint64_t make_sw128_mnmajor_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(FA_SUB >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// 2^x on the special-function unit (the softmax spends most of its instructions here).
__device__ __forceinline__ float fa_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ int fa_num_blocks(const FaParams& p, int q_tile) {
  int nblk = (p.Skv + FA_BN - 1) / FA_BN;
  if (p.causal) {
    const int last_q = p.q_offset + (q_tile + 1) * FA_BM - 1;  // last query position of the tile
    const int lim = last_q - p.kv_offset;                       // last visible key (local index)
    if (lim < 0) return 0;
    const int c = lim / FA_BN + 1;
    if (c < nblk) nblk = c;
  }
  return nblk;
}

__global__ void __launch_bounds__(FA_THREADS, 1) fa_fwd_kernel(const __grid_constant__ FaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem =
      reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + 2 * FA_SUB;       // [stage][2 sub-tiles]
  uint8_t* sV = sK + 4 * FA_SUB;
  uint8_t* sP = sV + 4 * FA_SUB;
  __shared__ FaCtl ctl;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const int q_tile = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int nblk = fa_num_blocks(p, q_tile);

  if (threadIdx.x == 0) {
    mbar_init(&ctl.q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl.k_full[i], 1);
      mbar_init(&ctl.v_full[i], 1);
      mbar_init(&ctl.kv_empty[i], 1);
      mbar_init(&ctl.s_full[i], 1);
      mbar_init(&ctl.s_empty[i], 4);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl.p_full[i], 4);
      mbar_init(&ctl.p_empty[i], 1);
      mbar_init(&ctl.pv_full[i], 1);
      mbar_init(&ctl.pv_empty[i], 4);
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
  const uint32_t tS[2] = {tmem, tmem + 128u};
  const uint32_t tPV[2] = {tmem + 256u, tmem + 384u};

  if (warp == 0) {
    if (lane == 0 && nblk > 0) {
      // ---------------------------------------------------------------- producer
      mbar_arrive_expect_tx(&ctl.q_full, 2 * FA_SUB);
      const int qrow = batch * p.Sq + q_tile * FA_BM;
      tma_load_3d(sQ, &p.tm_q, 0, head, qrow, &ctl.q_full);
      tma_load_3d(sQ + FA_SUB, &p.tm_q, 64, head, qrow, &ctl.q_full);
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&ctl.kv_empty[s], ((j >> 1) & 1) ^ 1u, &ctl.abort_flag, p.status, 0xA00 + s))
          break;
        const int krow = batch * p.Skv + j * FA_BN;
        mbar_arrive_expect_tx(&ctl.k_full[s], 2 * FA_SUB);
        tma_load_3d(sK + s * 2 * FA_SUB, &p.tm_k, 0, kv_head, krow, &ctl.k_full[s]);
        tma_load_3d(sK + s * 2 * FA_SUB + FA_SUB, &p.tm_k, 64, kv_head, krow, &ctl.k_full[s]);
        mbar_arrive_expect_tx(&ctl.v_full[s], 2 * FA_SUB);
        tma_load_3d(sV + s * 2 * FA_SUB, &p.tm_v, 0, kv_head, krow, &ctl.v_full[s]);
        tma_load_3d(sV + s * 2 * FA_SUB + FA_SUB, &p.tm_v, 64, kv_head, krow, &ctl.v_full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nblk > 0) {
      // --------------------------------------------------------------------- MMA
      constexpr uint32_t idesc_s = make_idesc(128, 128, 1u);
      constexpr uint32_t idesc_pv = make_idesc(128, 128, 1u) | (1u << 16);  // B is MN-major
      bool ok = mbar_wait(&ctl.q_full, 0, &ctl.abort_flag, p.status, 0xA10);
      auto issue_pv = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&ctl.p_full[s], ph, &ctl.abort_flag, p.status, 0xA20)) return false;
        if (!mbar_wait(&ctl.v_full[s], ph, &ctl.abort_flag, p.status, 0xA21)) return false;
        if (!mbar_wait(&ctl.pv_empty[s], ph ^ 1u, &ctl.abort_flag, p.status, 0xA22)) return false;
        tc_fence_after_sync();
        const uint32_t pa = smem_u32(sP + s * 2 * FA_SUB), va = smem_u32(sV + s * 2 * FA_SUB);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a_desc = make_sw128_kmajor_desc(pa + (kk >> 2) * FA_SUB) + 2u * (kk & 3);
          const uint64_t b_desc = make_sw128_mnmajor_desc(va + kk * 2048);
          mma_bf16_ss(tPV[s], a_desc, b_desc, idesc_pv, kk > 0 ? 1u : 0u);
        }
        mma_commit(&ctl.pv_full[s]);
        mma_commit(&ctl.kv_empty[s]);
        mma_commit(&ctl.p_empty[s]);
        return true;
      };
      for (int j = 0; ok && j < nblk; ++j) {
        const int s = j & 1;
        ok = mbar_wait(&ctl.k_full[s], (j >> 1) & 1, &ctl.abort_flag, p.status, 0xA11) &&
             mbar_wait(&ctl.s_empty[s], ((j >> 1) & 1) ^ 1u, &ctl.abort_flag, p.status, 0xA12);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + s * 2 * FA_SUB);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a_desc = make_sw128_kmajor_desc(qa + (kk >> 2) * FA_SUB) + 2u * (kk & 3);
          const uint64_t b_desc = make_sw128_kmajor_desc(ka + (kk >> 2) * FA_SUB) + 2u * (kk & 3);
          mma_bf16_ss(tS[s], a_desc, b_desc, idesc_s, kk > 0 ? 1u : 0u);
        }
        mma_commit(&ctl.s_full[s]);
        if (j > 0) ok = issue_pv(j - 1);
      }
      if (ok) issue_pv(nblk - 1);
    }
  } else {
    // ------------------------------------------------------------------- softmax
    const uint32_t q = warp & 3u;
    const uint32_t r = q * 32u + lane;  // query row of this thread inside the tile
    const uint32_t lane_addr = (q * 32u) << 16;
    const int q_pos = p.q_offset + q_tile * FA_BM + static_cast<int>(r);
    float o[FA_D];
#pragma unroll
    for (int i = 0; i < FA_D; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    // O += PV of block j is applied AFTER the softmax of block j+1, so the P*V MMA of block j
    // runs while these warps are busy with the next block instead of being waited for.
    auto o_update = [&](int j, float alpha) -> bool {
      const int b = j & 1;
      if (!mbar_wait(&ctl.pv_full[b], (j >> 1) & 1, &ctl.abort_flag, p.status, 0xA32)) return false;
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t p0[32], p1[32];
        tmem_ld_32x32(tPV[b] + lane_addr + c * 64u, p0);
        tmem_ld_32x32(tPV[b] + lane_addr + c * 64u + 32u, p1);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          o[c * 64 + i] = o[c * 64 + i] * alpha + __uint_as_float(p0[i]);
          o[c * 64 + 32 + i] = o[c * 64 + 32 + i] * alpha + __uint_as_float(p1[i]);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.pv_empty[b]);
      return true;
    };
    float alpha_prev = 1.f;
    bool ok = true;
    for (int j = 0; ok && j < nblk; ++j) {
      const int b = j & 1;
      if (!mbar_wait(&ctl.s_full[b], (j >> 1) & 1, &ctl.abort_flag, p.status, 0xA30)) { ok = false; break; }
      tc_fence_after_sync();
      const int key0 = p.kv_offset + j * FA_BN;   // global position of the block's first key
      const int kv_left = p.Skv - j * FA_BN;      // keys of this block that exist
      // Only blocks that touch the diagonal or the end of the keys need per-element masks.
      const bool need_mask = kv_left < FA_BN ||
                             (p.causal && key0 + FA_BN - 1 > p.q_offset + q_tile * FA_BM);
      // pass 1: row maximum (64 columns per TMEM round trip)
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t s0[32], s1[32];
        tmem_ld_32x32(tS[b] + lane_addr + c * 64u, s0);
        tmem_ld_32x32(tS[b] + lane_addr + c * 64u + 32u, s1);
        tmem_wait_ld();
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            mx = fmaxf(mx, fmaxf(__uint_as_float(s0[i]), __uint_as_float(s1[i])));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int k0 = c * 64 + i, k1 = k0 + 32;
            if (k0 < kv_left && (!p.causal || key0 + k0 <= q_pos)) mx = fmaxf(mx, __uint_as_float(s0[i]));
            if (k1 < kv_left && (!p.causal || key0 + k1 <= q_pos)) mx = fmaxf(mx, __uint_as_float(s1[i]));
          }
        }
      }
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m - m_use);  // m = -inf -> 0
      // pass 2: p = exp2(s*scale - m), row sum, bf16 P into shared memory
      if (!mbar_wait(&ctl.p_empty[b], ((j >> 1) & 1) ^ 1u, &ctl.abort_flag, p.status, 0xA31)) { ok = false; break; }
      uint8_t* sPb = sP + b * 2 * FA_SUB;
      float psum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t sr[32];
        tmem_ld_32x32(tS[b] + lane_addr + c * 32u, sr);
        tmem_wait_ld();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int kc = c * 32 + i;
          float p0 = fa_ex2(__uint_as_float(sr[i]) * p.scale_log2 - m_use);
          float p1 = fa_ex2(__uint_as_float(sr[i + 1]) * p.scale_log2 - m_use);
          if (need_mask) {
            if (!(kc < kv_left && (!p.causal || key0 + kc <= q_pos))) p0 = 0.f;
            if (!(kc + 1 < kv_left && (!p.causal || key0 + kc + 1 <= q_pos))) p1 = 0.f;
          }
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          // the row sum uses the rounded values, as the MMA will
          const float2 back = __bfloat1622float2(h);
          psum += back.x + back.y;
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
        }
        // 32 keys = four 16-byte chunks of the row; K-major sub-tile t = keys/64
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const uint32_t chunk = c * 4u + cc;            // 0..15 along the 128 keys
          const uint32_t t = chunk >> 3, ci = chunk & 7u;
          uint8_t* dst = sPb + t * FA_SUB + r * 128u + ((ci ^ (r & 7u)) * 16u);
          *reinterpret_cast<uint4*>(dst) = make_uint4(packed[cc * 4], packed[cc * 4 + 1],
                                                      packed[cc * 4 + 2], packed[cc * 4 + 3]);
        }
      }
      // S buffer free, P ready
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&ctl.s_empty[b]);
        mbar_arrive(&ctl.p_full[b]);
      }
      l = l * alpha + psum;
      m = m_new;
      if (j > 0) ok = o_update(j - 1, alpha_prev);
      alpha_prev = alpha;
    }
    if (ok && nblk > 0) o_update(nblk - 1, alpha_prev);
    // ------------------------------------------------------------------ epilogue
    const int row = q_tile * FA_BM + static_cast<int>(r);
    if (row < p.Sq) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst =
          p.o + ((static_cast<size_t>(batch) * p.Sq + row) * p.Hq + head) * FA_D;
#pragma unroll
      for (int i = 0; i < FA_D; i += 8) {
        uint4 v;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          h[k] = __floats2bfloat162_rn(o[i + 2 * k] * inv, o[i + 2 * k + 1] * inv);
        *reinterpret_cast<uint4*>(dst + i) = v;
      }
      p.lse[(static_cast<size_t>(batch) * p.Hq + head) * p.Sq + row] =
          l > 0.f ? (m * 0.6931471805599453f + logf(l)) : -INFINITY;
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

// Exact merge of two partial results over disjoint key sets:
//   acc (fp32 O, lse) <- merge(acc, part (bf16 O, lse)).  `first` initialises acc from part.
__global__ void attn_merge_kernel(float* __restrict__ o_acc, float* __restrict__ lse_acc,
                                  const __nv_bfloat16* __restrict__ o_part,
                                  const float* __restrict__ lse_part, int B, int S, int H,
                                  int first) {
  const long long total = static_cast<long long>(B) * S * H * (FA_D / 8);
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = idx % (FA_D / 8);
    long long t = idx / (FA_D / 8);
    const int h = t % H;
    t /= H;
    const int s = t % S;
    const int b = static_cast<int>(t / S);
    const size_t li = (static_cast<size_t>(b) * H + h) * S + s;
    const size_t oi = ((static_cast<size_t>(b) * S + s) * H + h) * FA_D + v * 8;
    const float lp = lse_part[li];
    const float la = first ? -INFINITY : lse_acc[li];
    const float mx = fmaxf(lp, la);
    float wa = 0.f, wp = 0.f, ln = -INFINITY;
    if (mx > -INFINITY) {
      const float ea = __expf(la - mx), ep = __expf(lp - mx);
      wa = ea / (ea + ep);
      wp = ep / (ea + ep);
      ln = mx + __logf(ea + ep);
    }
    const uint4 raw = *reinterpret_cast<const uint4*>(o_part + oi);
    const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float4 a0 = first ? make_float4(0, 0, 0, 0) : *reinterpret_cast<float4*>(o_acc + oi);
    float4 a1 = first ? make_float4(0, 0, 0, 0) : *reinterpret_cast<float4*>(o_acc + oi + 4);
    const float2 p0 = __bfloat1622float2(hp[0]), p1 = __bfloat1622float2(hp[1]),
                 p2 = __bfloat1622float2(hp[2]), p3 = __bfloat1622float2(hp[3]);
    a0 = make_float4(a0.x * wa + p0.x * wp, a0.y * wa + p0.y * wp, a0.z * wa + p1.x * wp,
                     a0.w * wa + p1.y * wp);
    a1 = make_float4(a1.x * wa + p2.x * wp, a1.y * wa + p2.y * wp, a1.z * wa + p3.x * wp,
                     a1.w * wa + p3.y * wp);
    *reinterpret_cast<float4*>(o_acc + oi) = a0;
    *reinterpret_cast<float4*>(o_acc + oi + 4) = a1;
    if (v == 0) lse_acc[li] = ln;
  }
}

}  // namespace cb

using namespace cb;

static int make_tmap_bshd(CUtensorMap* out, const void* base, int rows, int heads) {
  const DriverApi& d = driver_api();
  if (!d.ok) {
    set_last_error("tensor map: " + d.why);
    return -1;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) {
    set_last_error("attention: tensors must be 16-byte aligned");
    return -1;
  }
  cuuint64_t dims[3] = {FA_D, static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[2] = {FA_D * 2ull, static_cast<cuuint64_t>(heads) * FA_D * 2ull};
  cuuint32_t box[3] = {64, 1, 128};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = d.cuTensorMapEncodeTiled(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                                        const_cast<void*>(base), dims, strides, box, estr,
                                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuTensorMapEncodeTiled(attention)", r));
    return -1;
  }
  return 0;
}

// Shared with the other attention kernels of this folder.
int cb_attn_make_tmap_bshd(CUtensorMap* out, const void* base, int rows, int heads) {
  return make_tmap_bshd(out, base, rows, heads);
}

extern "C" {

// q [B, Sq, Hq, 128], k/v [B, Skv, Hkv, 128], o [B, Sq, Hq, 128] bf16 contiguous;
// lse [B, Hq, Sq] fp32.  q_offset / kv_offset are the global sequence positions of the
// first query row / key (they only matter for the causal mask).
int cb_attn_fwd(const void* q, const void* k, const void* v, void* o, void* lse, int B, int Sq,
                int Skv, int Hq, int Hkv, int q_offset, int kv_offset, int causal, float scale,
                void* status, void* stream) {
  if (B < 1 || Sq < 1 || Skv < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0) {
    set_last_error("attention: bad shape (Hq must be a multiple of Hkv)");
    return -1;
  }
  FaParams p;
  if (make_tmap_bshd(&p.tm_q, q, B * Sq, Hq)) return -1;
  if (make_tmap_bshd(&p.tm_k, k, B * Skv, Hkv)) return -1;
  if (make_tmap_bshd(&p.tm_v, v, B * Skv, Hkv)) return -1;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = static_cast<float*>(lse);
  p.B = B;
  p.Sq = Sq;
  p.Skv = Skv;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.q_offset = q_offset;
  p.kv_offset = kv_offset;
  p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = static_cast<uint32_t*>(status);
  cudaError_t e = cudaFuncSetAttribute(fa_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       FA_SMEM);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    return -1;
  }
  dim3 grid((Sq + FA_BM - 1) / FA_BM, Hq, B);
  fa_fwd_kernel<<<grid, FA_THREADS, FA_SMEM, static_cast<cudaStream_t>(stream)>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(std::string("attention launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

int cb_attn_merge(void* o_acc, void* lse_acc, const void* o_part, const void* lse_part, int B,
                  int S, int H, int first, void* stream) {
  attn_merge_kernel<<<1184, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<float*>(o_acc), static_cast<float*>(lse_acc),
      static_cast<const __nv_bfloat16*>(o_part), static_cast<const float*>(lse_part), B, S, H,
      first);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
