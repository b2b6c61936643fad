// Collective kernels over symmetric memory: all-reduce (one-shot pull,
// two-shot reduce-scatter + all-gather, NVLS multimem), all-gather,
// reduce-scatter, all-to-all (flat and 4-D sequence<->head), broadcast, barrier.
// Each is ONE launch: the cross-GPU barriers that the reference issues as
// separate <<<1,1>>> kernels around its collectives
// (datasets/example048_thunderkitten_all_reduce_easy/nv/
// empty_thunderkitten_all_reduce.cu:291-315) are folded into the kernel, per CTA,
// on the CTA's own signal-pad channel.
//
// Designs and where the reference has the same capability:
//  * one-shot pull all-reduce : datasets/example105_sglang_custom_allreduce_easy/
//    empty_sglang_custom_allreduce_pull_easy.cu:49-111 (every CTA reads all ranks'
//    16-byte vectors, reduces in fp32);
//  * two-shot                  : reduce-scatter then all-gather, the "rsag" structure of
//    datasets/example031_msclpp_allreduce_rsag_zero_easy/empty_mscclpp_allreduce_easy.cu:186-224
//    without a host proxy, and vLLM's two-shot custom all-reduce
//    (datasets/example097_vllm_custom_all_reduce/nv/empty_vllm_custom_all_reduce.py:104-145);
//  * NVLS                      : multimem.ld_reduce + multimem.st, each rank owning 1/W of the
//    vectors (datasets/example048_thunderkitten_all_reduce_easy/nv/
//    empty_thunderkitten_all_reduce.cu:64-94);
//  * all-gather / reduce-scatter / all-to-all : datasets/example030_mscclpp_allgather_fullmesh_easy/
//    empty_mscclpp_allgather.cu:136-154, datasets/example050_thunderkitten_reduce_scatter_easy/nv/
//    empty_thunderkitten_reduce_scatter.cu:64-95, datasets/example049_thunderkitten_alltoall_easy/nv/
//    empty_thunderkitten_alltoall.cu:60-121, datasets/example018_mscclpp_alltoall_easy/
//    empty_mscclpp_all2all_easy.cu:117-120;
//  * broadcast                 : datasets/example034_nvshmem_broadcast/nv/
//    empty_nvshmem_broadcast.cu:101-118.
//
// Work split: CTA b of every rank works on slice b of the message, and only
// ever depends on CTA b of the peers, so a per-CTA channel barrier is enough and
// no grid-wide barrier is needed.  Grids never exceed one resident wave.
#include "coll_common.cuh"

namespace cb {

enum : uint32_t { PH_COPY_IN = 16, PH_REDUCE = 17, PH_GATHER = 18 };

static constexpr int kCollThreads = 512;

// ---------------------------------------------------------------- local copies
__device__ __forceinline__ void copy_vec_slice(void* dst, const void* src, unsigned long long v0,
                                               unsigned long long v1) {
  const uint4* s = static_cast<const uint4*>(src);
  uint4* d = static_cast<uint4*>(dst);
  unsigned long long i = v0 + threadIdx.x;
  for (; i + 3ull * blockDim.x < v1; i += 4ull * blockDim.x) {
    uint4 a = s[i], b = s[i + blockDim.x], c = s[i + 2ull * blockDim.x],
          e = s[i + 3ull * blockDim.x];
    d[i] = a;
    d[i + blockDim.x] = b;
    d[i + 2ull * blockDim.x] = c;
    d[i + 3ull * blockDim.x] = e;
  }
  for (; i < v1; i += blockDim.x) d[i] = s[i];
}

// Bandwidth loop over vectors [begin, end) of one CTA: every thread issues U independent
// loads and only then the U stores, so U 16-byte requests per thread are in flight.  The
// latency of a peer or multicast load is a few microseconds, so bytes in flight decide the
// rate.  `load(i)` returns vector i, `store(i, v)` writes it.
template <int U, class L, class S>
__device__ __forceinline__ void span_copy_fixed(unsigned long long begin, unsigned long long end,
                                                L load, S store) {
  const unsigned long long st = blockDim.x;
  unsigned long long i = begin + threadIdx.x;
  for (; i + static_cast<unsigned long long>(U - 1) * st < end;
       i += static_cast<unsigned long long>(U) * st) {
    uint4 r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) r[u] = load(i + static_cast<unsigned long long>(u) * st);
#pragma unroll
    for (int u = 0; u < U; ++u) store(i + static_cast<unsigned long long>(u) * st, r[u]);
  }
  for (; i < end; i += st) store(i, load(i));
}
// `unroll` is uniform over the grid (it comes from the argument block).
template <class L, class S>
__device__ __forceinline__ void span_copy(int unroll, unsigned long long begin,
                                          unsigned long long end, L load, S store) {
  if (unroll >= 8)
    span_copy_fixed<8>(begin, end, load, store);
  else if (unroll >= 4 || unroll <= 0)
    span_copy_fixed<4>(begin, end, load, store);
  else
    span_copy_fixed<2>(begin, end, load, store);
}

// Copies bytes [16*v0, min(16*v1, nbytes)) of an arbitrary local tensor into /
// out of a 16-byte padded symmetric buffer; the ragged tail goes byte-wise.
__device__ __forceinline__ void copy_bytes_slice(void* dst, const void* src,
                                                 unsigned long long nbytes, unsigned long long v0,
                                                 unsigned long long v1, bool zero_pad_dst) {
  const unsigned long long full = nbytes / 16ull;
  const unsigned long long v1f = v1 < full ? v1 : full;
  if (v0 < v1f) copy_vec_slice(dst, src, v0, v1f);
  if (v1 > full && v0 <= full && threadIdx.x == 0) {
    const unsigned char* s = static_cast<const unsigned char*>(src);
    unsigned char* d = static_cast<unsigned char*>(dst);
    for (unsigned long long i = full * 16ull; i < nbytes; ++i) d[i] = s[i];
    if (zero_pad_dst)
      for (unsigned long long i = nbytes; i < (full + 1ull) * 16ull; ++i) d[i] = 0;
  }
}

// The per-channel rank barrier only orders block b of this rank against block b of
// every peer.  So whatever block b of a PEER reads from this rank after the barrier must
// have been written here by block b itself.  Algorithms that split the message into W rank
// chunks and then split each chunk over the grid read "slice b of chunk <their rank>":
// staging copies therefore walk slice b of EVERY chunk, not slice b of the whole message.
template <class F>
__device__ __forceinline__ void for_each_chunk_slice(unsigned long long nvec,
                                                     unsigned long long per_rank, int world, F f) {
  for (int r = 0; r < world; ++r) {
    unsigned long long c0 = per_rank * r, c1 = c0 + per_rank;
    if (c0 > nvec) c0 = nvec;
    if (c1 > nvec) c1 = nvec;
    unsigned long long s0, s1;
    slice_of(c1 - c0, gridDim.x, blockIdx.x, &s0, &s1);
    if (s1 > s0) f(c0 + s0, c0 + s1);
  }
}

__device__ __forceinline__ uint32_t begin_epoch(const CbComm& c, uint32_t ch) {
  // Every thread reads the same word; no thread writes it before end_epoch's barrier.
  const uint32_t e = ld_volatile(c.epoch + ch);
  if (c.jitter_ns != 0u) {  // debug stress: a different, repeatable delay per (rank, CTA, call)
    uint32_t h = (static_cast<uint32_t>(c.rank) * 0x9e3779b9u) ^ (blockIdx.x * 0x85ebca6bu) ^
                 (e * 0xc2b2ae35u);
    h ^= h >> 15;
    h *= 0x2c1b3c6du;
    h ^= h >> 12;
    uint32_t left = h % c.jitter_ns;
    while (left > 0u) {  // one __nanosleep is capped near a millisecond
      const uint32_t step = left < 500000u ? left : 500000u;
      __nanosleep(step);
      left -= step;
    }
  }
  return e;
}
__device__ __forceinline__ void end_epoch(const CbComm& c, uint32_t ch, uint32_t value) {
  __syncthreads();
  if (threadIdx.x == 0) c.epoch[ch] = value;
}

// Sum over the W ranks of vector (off + i) for i in [begin, end), pulled with system-scope
// loads.  raw[r] comes from rank r and the sum runs in rank order 0..W-1, so every rank
// rounds alike; the indices are compile-time constants, so the vectors stay in registers.
// U vectors x W ranks are in flight per thread; `store(i, v)` takes the sum.
template <int DT, int W>
__device__ __forceinline__ uint4 sum_in_rank_order(const uint4 (&raw)[W]) {
  float acc[Vec16<DT>::N];
#pragma unroll
  for (int r = 0; r < W; ++r) {
    float f[Vec16<DT>::N];
    Vec16<DT>::unpack(raw[r], f);
#pragma unroll
    for (int k = 0; k < Vec16<DT>::N; ++k) acc[k] = (r == 0) ? f[k] : acc[k] + f[k];
  }
  return Vec16<DT>::pack(acc);
}
template <int DT, int W, int U, class S>
__device__ __forceinline__ void reduce_span_fixed(const CollArgs& a, unsigned long long off,
                                                  unsigned long long begin,
                                                  unsigned long long end, S store) {
  const unsigned long long st = blockDim.x;
  const uint4* base[W];
#pragma unroll
  for (int r = 0; r < W; ++r) base[r] = static_cast<const uint4*>(a.sym[r]) + off;
  unsigned long long i = begin + threadIdx.x;
  for (; i + static_cast<unsigned long long>(U - 1) * st < end;
       i += static_cast<unsigned long long>(U) * st) {
    uint4 raw[U][W];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int r = 0; r < W; ++r)
        raw[u][r] = ld_sys_v4(base[r] + i + static_cast<unsigned long long>(u) * st);
#pragma unroll
    for (int u = 0; u < U; ++u)
      store(i + static_cast<unsigned long long>(u) * st, sum_in_rank_order<DT, W>(raw[u]));
  }
  for (; i < end; i += st) {
    uint4 raw[W];
#pragma unroll
    for (int r = 0; r < W; ++r) raw[r] = ld_sys_v4(base[r] + i);
    store(i, sum_in_rank_order<DT, W>(raw));
  }
}
// Runtime choice of U: at most 16 loads per thread (register budget of a 512-thread CTA),
// eight by default.
template <int DT, int W, class S>
__device__ __forceinline__ void reduce_span(const CollArgs& a, unsigned long long off,
                                            unsigned long long begin, unsigned long long end,
                                            S store) {
  constexpr int UMAX = (W >= 16) ? 1 : (16 / W > 8 ? 8 : 16 / W);
  constexpr int UDEF = (W >= 8) ? 1 : 8 / W;
  const int u = a.unroll <= 0 ? UDEF : a.unroll;
  if constexpr (UMAX >= 4) {
    if (u >= UMAX)
      reduce_span_fixed<DT, W, UMAX>(a, off, begin, end, store);
    else if (u >= UMAX / 2)
      reduce_span_fixed<DT, W, UMAX / 2>(a, off, begin, end, store);
    else
      reduce_span_fixed<DT, W, UMAX / 4>(a, off, begin, end, store);
  } else if constexpr (UMAX == 2) {
    if (u >= 2)
      reduce_span_fixed<DT, W, 2>(a, off, begin, end, store);
    else
      reduce_span_fixed<DT, W, 1>(a, off, begin, end, store);
  } else {
    reduce_span_fixed<DT, W, 1>(a, off, begin, end, store);
  }
}

// ------------------------------------------------------------ one-shot pull AR
template <int DT, int W>
__global__ void __launch_bounds__(kCollThreads)
    ar_oneshot_kernel(const __grid_constant__ CollArgs args, const CollArgs* emu) {
  const CollArgs& a = pick_args(args, emu);
  const CbComm& c = a.comm;
  const uint32_t ch = cta_channel(0);
  const uint32_t e = begin_epoch(c, ch);
  const unsigned long long nvec = (a.nbytes + 15ull) / 16ull;
  unsigned long long v0, v1;
  slice_of(nvec, gridDim.x, blockIdx.x, &v0, &v1);

  if (a.copy_in) copy_bytes_slice(a.sym[c.rank], a.in, a.nbytes, v0, v1, true);
  bool ok = rank_barrier_block(c, ch, e + 1, PH_BARRIER_START);
  if (ok) {
    // The result never goes to sym[rank]: peers may still be reading it.  `out` is an
    // ordinary local tensor (the host wrapper guarantees it does not alias sym[rank]).
    uint4* out = static_cast<uint4*>(a.out);
    const unsigned long long full = a.nbytes / 16ull;
    for (unsigned long long i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
      float acc[Vec16<DT>::N];
      uint4 raw[W];
#pragma unroll
      for (int p = 0; p < W; ++p) {
        // Start at the own copy and rotate so the W ranks do not gang up on one peer.
        const int src = (c.rank + p) % W;
        raw[p] = ld_sys_v4(static_cast<const uint4*>(a.sym[src]) + i);
      }
      // Sum in rank order so every rank produces the same bits.
#pragma unroll
      for (int r = 0; r < W; ++r) {
        const int p = (r - c.rank + W) % W;
        float f[Vec16<DT>::N];
        Vec16<DT>::unpack(raw[p], f);
#pragma unroll
        for (int k = 0; k < Vec16<DT>::N; ++k) acc[k] = (r == 0) ? f[k] : acc[k] + f[k];
      }
      const uint4 res = Vec16<DT>::pack(acc);
      if (i < full) {
        out[i] = res;
      } else {
        const unsigned char* s = reinterpret_cast<const unsigned char*>(&res);
        unsigned char* d = reinterpret_cast<unsigned char*>(a.out) + i * 16ull;
        for (unsigned long long k = 0; k < a.nbytes - i * 16ull; ++k) d[k] = s[k];
      }
    }
    // Peers must be done reading sym[rank] before a later launch overwrites it.
    ok = rank_barrier_block(c, ch, e + 2, PH_BARRIER_END);
  }
  end_epoch(c, ch, e + 2);
}

// --------------------------------------------------------------- two-shot AR
// Phase 1: rank r sums chunk r over all ranks (pull) and writes it back into its
// own symmetric buffer.  Phase 2: every rank pulls the W reduced chunks.
template <int DT, int W>
__global__ void __launch_bounds__(kCollThreads)
    ar_twoshot_kernel(const __grid_constant__ CollArgs args, const CollArgs* emu) {
  const CollArgs& a = pick_args(args, emu);
  const CbComm& c = a.comm;
  const uint32_t ch = cta_channel(0);
  const uint32_t e = begin_epoch(c, ch);
  const unsigned long long nvec = (a.nbytes + 15ull) / 16ull;
  const unsigned long long per_rank = (nvec + W - 1) / W;
  const bool push = (a.variant & 1) != 0;

  if (a.copy_in)
    for_each_chunk_slice(nvec, per_rank, W, [&](unsigned long long v0, unsigned long long v1) {
      copy_bytes_slice(a.sym[c.rank], a.in, a.nbytes, v0, v1, true);
    });
  bool ok = rank_barrier_block(c, ch, e + 1, PH_BARRIER_START);
  if (ok) {
    // Phase 1 on my chunk.
    unsigned long long c0 = per_rank * c.rank, c1 = c0 + per_rank;
    if (c0 > nvec) c0 = nvec;
    if (c1 > nvec) c1 = nvec;
    unsigned long long s0, s1;
    slice_of(c1 - c0, gridDim.x, blockIdx.x, &s0, &s1);
    if (push) {
      // Each sum goes to every rank at once: no second phase.  A vector is read and later
      // overwritten by the same thread, and no other rank touches chunk `rank`.
      reduce_span<DT, W>(a, 0, c0 + s0, c0 + s1, [&](unsigned long long i, uint4 v) {
#pragma unroll
        for (int r = 0; r < W; ++r) st_sys_v4(static_cast<uint4*>(a.sym[r]) + i, v);
      });
    } else {
      reduce_span<DT, W>(a, 0, c0 + s0, c0 + s1, [&](unsigned long long i, uint4 v) {
        st_sys_v4(static_cast<uint4*>(a.sym[c.rank]) + i, v);
      });
    }
    ok = rank_barrier_block(c, ch, e + 2, PH_BARRIER_MID);  // its release orders the stores
  }
  if (ok && push) {
    // Slice b of every chunk was written here by block b of that chunk's owner.
    if (a.copy_out)
      for_each_chunk_slice(nvec, per_rank, W, [&](unsigned long long v0, unsigned long long v1) {
        copy_bytes_slice(a.out, a.sym[c.rank], a.nbytes, v0, v1, false);
      });
    // Keeps the epoch arithmetic of the pull form: nobody waits on e + 3 later, the next
    // call starts from the stored epoch.
  } else if (ok) {
    // Phase 2: gather slice b of every rank's reduced chunk.
    unsigned char* outb = static_cast<unsigned char*>(a.copy_out ? a.out : a.sym[c.rank]);
    const unsigned long long full = a.nbytes / 16ull;
#pragma unroll 1
    for (int p = 0; p < W; ++p) {
      const int src = (c.rank + p) % W;
      if (!a.copy_out && src == c.rank) continue;  // already in place
      unsigned long long c0 = per_rank * src, c1 = c0 + per_rank;
      if (c0 > nvec) c0 = nvec;
      if (c1 > nvec) c1 = nvec;
      unsigned long long s0, s1;
      slice_of(c1 - c0, gridDim.x, blockIdx.x, &s0, &s1);
      const uint4* sp = static_cast<const uint4*>(a.sym[src]);
      // Whole vectors first; the vector that holds the ragged tail goes through the slow loop.
      const unsigned long long vend = (c0 + s1 < full) ? c0 + s1 : (full > c0 + s0 ? full : c0 + s0);
      uint4* d = reinterpret_cast<uint4*>(outb);
      span_copy(
          a.unroll, c0 + s0, vend, [&](unsigned long long i) { return ld_sys_v4(sp + i); },
          [&](unsigned long long i, uint4 v) { d[i] = v; });
      for (unsigned long long i = vend + threadIdx.x; i < c0 + s1; i += blockDim.x) {
        const uint4 v = ld_sys_v4(sp + i);
        if (i < full || !a.copy_out) {
          *reinterpret_cast<uint4*>(outb + i * 16ull) = v;
        } else {
          const unsigned char* s = reinterpret_cast<const unsigned char*>(&v);
          for (unsigned long long k = 0; k < a.nbytes - i * 16ull; ++k) outb[i * 16ull + k] = s[k];
        }
      }
    }
    ok = rank_barrier_block(c, ch, e + 3, PH_BARRIER_END);
  }
  end_epoch(c, ch, e + 3);
}

// ------------------------------------------------------------------- NVLS AR
// Rank r owns 1/W of the vectors: one multimem.ld_reduce returns the sum over
// all ranks (added inside the switch), one multimem.st writes it to all ranks.
template <int DT, int W>
__global__ void __launch_bounds__(kCollThreads)
    ar_nvls_kernel(const __grid_constant__ CollArgs args, const CollArgs* emu) {
  const CollArgs& a = pick_args(args, emu);
  const CbComm& c = a.comm;
  const uint32_t ch = cta_channel(0);
  const uint32_t e = begin_epoch(c, ch);
  const unsigned long long nvec = (a.nbytes + 15ull) / 16ull;
  const unsigned long long per_rank = (nvec + W - 1) / W;
  if (a.copy_in)
    for_each_chunk_slice(nvec, per_rank, W, [&](unsigned long long v0, unsigned long long v1) {
      copy_bytes_slice(a.sym[c.rank], a.in, a.nbytes, v0, v1, true);
    });
  bool ok = rank_barrier_block(c, ch, e + 1, PH_BARRIER_START);
  if (ok) {
    unsigned long long c0 = per_rank * c.rank, c1 = c0 + per_rank;
    if (c0 > nvec) c0 = nvec;
    if (c1 > nvec) c1 = nvec;
    unsigned long long s0, s1;
    slice_of(c1 - c0, gridDim.x, blockIdx.x, &s0, &s1);
    uint4* mc = static_cast<uint4*>(a.mc);
    span_copy(
        a.unroll, c0 + s0, c0 + s1,
        [&](unsigned long long i) { return Vec16<DT>::mm_reduce(mc + i); },
        [&](unsigned long long i, uint4 v) { mm_st_v4(mc + i, v); });
    // multimem.st results must be visible on every rank before anyone reads them: the
    // barrier's CTA sync followed by its release stores orders them (a system fence by
    // every thread here costs tens of microseconds under store traffic).
    ok = rank_barrier_block(c, ch, e + 2, PH_BARRIER_END);
  }
  // Slice b of every chunk was written by block b of that chunk's owner: safe to read now.
  if (ok && a.copy_out)
    for_each_chunk_slice(nvec, per_rank, W, [&](unsigned long long v0, unsigned long long v1) {
      copy_bytes_slice(a.out, a.sym[c.rank], a.nbytes, v0, v1, false);
    });
  end_epoch(c, ch, e + 2);
}

// ---------------------------------------------------------------- all-gather
// nbytes = bytes of ONE rank's shard.  Output = W shards in rank order.
// Pull form: shards are staged in symmetric memory (copy_in) or already there;
// rank r's shard sits at byte offset r*shard_stride of ITS OWN buffer only when
// `in` aliases the output; here every rank stages at offset 0.
template <int W>
__global__ void __launch_bounds__(kCollThreads)
    ag_pull_kernel(const __grid_constant__ CollArgs args, const CollArgs* emu) {
  const CollArgs& a = pick_args(args, emu);
  const CbComm& c = a.comm;
  const uint32_t ch = cta_channel(0);
  const uint32_t e = begin_epoch(c, ch);
  const unsigned long long nvec = (a.nbytes + 15ull) / 16ull;
  unsigned long long v0, v1;
  slice_of(nvec, gridDim.x, blockIdx.x, &v0, &v1);
  if (a.copy_in) copy_bytes_slice(a.sym[c.rank], a.in, a.nbytes, v0, v1, true);
  bool ok = rank_barrier_block(c, ch, e + 1, PH_BARRIER_START);
  if (ok) {
    unsigned char* outb = static_cast<unsigned char*>(a.out);
    const bool aligned = (a.nbytes % 16ull) == 0;
#pragma unroll 1
    for (int p = 0; p < W; ++p) {
      const int src = (c.rank + p) % W;
      const uint4* sp = static_cast<const uint4*>(a.sym[src]);
      unsigned char* dst = outb + a.nbytes * src;
      if (aligned) {
        uint4* d = reinterpret_cast<uint4*>(dst);
        span_copy(
            a.unroll, v0, v1, [&](unsigned long long i) { return ld_sys_v4(sp + i); },
            [&](unsigned long long i, uint4 v) { d[i] = v; });
      } else {
        // Shard size not a multiple of 16 B: destinations are unaligned, go 4 bytes / 1 byte.
        const unsigned long long b0 = v0 * 16ull;
        unsigned long long b1 = v1 * 16ull;
        if (b1 > a.nbytes) b1 = a.nbytes;
        const unsigned char* s = reinterpret_cast<const unsigned char*>(sp);
        for (unsigned long long i = b0 + threadIdx.x; i < b1; i += blockDim.x) dst[i] = s[i];
      }
    }
    ok = rank_barrier_block(c, ch, e + 2, PH_BARRIER_END);
  }
  end_epoch(c, ch, e + 2);
}

// Push form into a symmetric OUTPUT (sym[] is the gathered tensor, W*nbytes per
// rank): every rank stores its shard at offset rank*nbytes of every peer, either
// with one multimem.st per vector (mc != nullptr) or with W plain stores.
template <int W>
__global__ void __launch_bounds__(kCollThreads)
    ag_push_kernel(const __grid_constant__ CollArgs args, const CollArgs* emu) {
  const CollArgs& a = pick_args(args, emu);
  const CbComm& c = a.comm;
  const uint32_t ch = cta_channel(0);
  const uint32_t e = begin_epoch(c, ch);
  const unsigned long long nvec = a.nbytes / 16ull;  // host guarantees a multiple of 16
  unsigned long long v0, v1;
  slice_of(nvec, gridDim.x, blockIdx.x, &v0, &v1);
  // Peers must have finished reading the previous contents of the output.
  bool ok = rank_barrier_block(c, ch, e + 1, PH_BARRIER_START);
  if (ok) {
    const uint4* src = static_cast<const uint4*>(a.in);
    const unsigned long long off = nvec * c.rank;
    if (a.mc != nullptr) {
      uint4* mc = static_cast<uint4*>(a.mc) + off;
      span_copy(
          a.unroll, v0, v1, [&](unsigned long long i) { return src[i]; },
          [&](unsigned long long i, uint4 v) { mm_st_v4(mc + i, v); });
    } else {
      span_copy(
          a.unroll, v0, v1, [&](unsigned long long i) { return src[i]; },
          [&](unsigned long long i, uint4 v) {
#pragma unroll
            for (int p = 0; p < W; ++p) {
              const int dst = (c.rank + p) % W;
              st_sys_v4(static_cast<uint4*>(a.sym[dst]) + off + i, v);
            }
          });
    }
    ok = rank_barrier_block(c, ch, e + 2, PH_BARRIER_END);  // its release orders the stores
  }
  end_epoch(c, ch, e + 2);
}

// ------------------------------------------------------------ reduce-scatter
// nbytes = bytes of the FULL input (W chunks); rank r outputs the sum of chunk r.
template <int DT, int W>
__global__ void __launch_bounds__(kCollThreads)
    rs_kernel(const __grid_constant__ CollArgs args, const CollArgs* emu) {
  const CollArgs& a = pick_args(args, emu);
  const CbComm& c = a.comm;
  const uint32_t ch = cta_channel(0);
  const uint32_t e = begin_epoch(c, ch);
  const unsigned long long nvec = a.nbytes / 16ull;  // host guarantees chunk % 16 == 0
  const unsigned long long per_rank = nvec / W;
  if (a.copy_in)
    for_each_chunk_slice(nvec, per_rank, W, [&](unsigned long long v0, unsigned long long v1) {
      copy_vec_slice(a.sym[c.rank], a.in, v0, v1);
    });
  bool ok = rank_barrier_block(c, ch, e + 1, PH_BARRIER_START);
  if (ok) {
    const unsigned long long c0 = per_rank * c.rank;
    unsigned long long s0, s1;
    slice_of(per_rank, gridDim.x, blockIdx.x, &s0, &s1);
    uint4* out = static_cast<uint4*>(a.out);
    if (a.mc != nullptr) {
      const uint4* mc = static_cast<const uint4*>(a.mc) + c0;
      span_copy(
          a.unroll, s0, s1, [&](unsigned long long i) { return Vec16<DT>::mm_reduce(mc + i); },
          [&](unsigned long long i, uint4 v) { out[i] = v; });
    } else {
      reduce_span<DT, W>(a, c0, s0, s1, [&](unsigned long long i, uint4 v) { out[i] = v; });
    }
    ok = rank_barrier_block(c, ch, e + 2, PH_BARRIER_END);
  }
  end_epoch(c, ch, e + 2);
}

// ---------------------------------------------------------------- all-to-all
// Flat: nbytes = bytes of the full per-rank input (W equal chunks);
// out chunk p <- chunk `rank` of rank p's input (pull).
template <int W>
__global__ void __launch_bounds__(kCollThreads)
    a2a_flat_kernel(const __grid_constant__ CollArgs args, const CollArgs* emu) {
  const CollArgs& a = pick_args(args, emu);
  const CbComm& c = a.comm;
  const uint32_t ch = cta_channel(0);
  const uint32_t e = begin_epoch(c, ch);
  const unsigned long long nvec = a.nbytes / 16ull;
  const unsigned long long per_rank = nvec / W;
  unsigned long long s0, s1;
  slice_of(per_rank, gridDim.x, blockIdx.x, &s0, &s1);
  if (a.variant & 1) {
    // Push form: sym[] is the (symmetric or staging) OUTPUT; chunk p of the local `in` is
    // stored into slot `rank` of rank p.  Plain stores need no request in the other direction.
    // Peers must have finished with the previous contents of their output first.
    bool ok = rank_barrier_block(c, ch, e + 1, PH_BARRIER_START);
    if (ok) {
      const uint4* in = static_cast<const uint4*>(a.in);
#pragma unroll 1
      for (int p = 0; p < W; ++p) {
        const int dst = (c.rank + p) % W;
        const uint4* sp = in + per_rank * dst;
        uint4* dp = static_cast<uint4*>(a.sym[dst]) + per_rank * c.rank;
        span_copy(
            a.unroll, s0, s1, [&](unsigned long long i) { return sp[i]; },
            [&](unsigned long long i, uint4 v) { st_sys_v4(dp + i, v); });
      }
      ok = rank_barrier_block(c, ch, e + 2, PH_BARRIER_END);  // its release orders the stores
    }
    // Slice b of every slot was written here by block b of the slot's rank.
    if (ok && a.copy_out)
      for_each_chunk_slice(nvec, per_rank, W, [&](unsigned long long v0, unsigned long long v1) {
        copy_vec_slice(a.out, a.sym[c.rank], v0, v1);
      });
    end_epoch(c, ch, e + 2);
    return;
  }
  if (a.copy_in)
    for_each_chunk_slice(nvec, per_rank, W, [&](unsigned long long v0, unsigned long long v1) {
      copy_vec_slice(a.sym[c.rank], a.in, v0, v1);
    });
  bool ok = rank_barrier_block(c, ch, e + 1, PH_BARRIER_START);
  if (ok) {
    uint4* out = static_cast<uint4*>(a.out);
#pragma unroll 1
    for (int p = 0; p < W; ++p) {
      const int src = (c.rank + p) % W;
      const uint4* sp = static_cast<const uint4*>(a.sym[src]) + per_rank * c.rank;
      uint4* dp = out + per_rank * src;
      span_copy(
          a.unroll, s0, s1, [&](unsigned long long i) { return ld_sys_v4(sp + i); },
          [&](unsigned long long i, uint4 v) { dp[i] = v; });
    }
    ok = rank_barrier_block(c, ch, e + 2, PH_BARRIER_END);
  }
  end_epoch(c, ch, e + 2);
}

// 4-D sequence<->head exchange (the Ulysses layouts), pull form.
//  to_heads = 1:  in [B, S/W, H, D]  -> out [B, S, H/W, D]
//                 out[b, p*Sl + s, h, :] = in_p[b, s, rank*Hl + h, :]
//  to_heads = 0:  in [B, S, H/W, D]  -> out [B, S/W, H, D]
//                 out[b, s, p*Hl + h, :] = in_p[b, rank*Sl + s, h, :]
// Rows of D elements are moved as 16-byte vectors (D * elem_size % 16 == 0).
template <int W>
__global__ void __launch_bounds__(kCollThreads)
    a2a_4d_kernel(const __grid_constant__ CollArgs args, const CollArgs* emu) {
  const CollArgs& a = pick_args(args, emu);
  const CbComm& c = a.comm;
  const uint32_t ch = cta_channel(0);
  const uint32_t e = begin_epoch(c, ch);
  const unsigned long long nvec = a.nbytes / 16ull;  // full per-rank input
  unsigned long long v0, v1;
  slice_of(nvec, gridDim.x, blockIdx.x, &v0, &v1);
  const unsigned long long B = a.a2a_b, Sl = a.a2a_s_local, H = a.a2a_h;
  const unsigned long long Hl = H / W;
  const unsigned long long dv = nvec / (B * Sl * H);  // vectors per D-row
  const unsigned long long run = Hl * dv;              // contiguous vectors per (b, s) and peer
  // Source offset of item (b, s, j) as read by rank `reader`.
  auto src_offset = [&](unsigned long long b, unsigned long long s, unsigned long long j,
                        int reader) -> unsigned long long {
    return a.a2a_to_heads
               ? ((b * Sl + s) * H + static_cast<unsigned long long>(reader) * Hl) * dv + j
               : ((b * (Sl * W) + static_cast<unsigned long long>(reader) * Sl + s) * Hl) * dv + j;
  };
  if (a.copy_in) {
    // Stage exactly the vectors that block b of each peer will read from this rank: item
    // idx = (p, b, s, j) is read from here by rank (rank - p) mod W.
    const uint4* in = static_cast<const uint4*>(a.in);
    uint4* mine = static_cast<uint4*>(a.sym[c.rank]);
    for (unsigned long long idx = v0 + threadIdx.x; idx < v1; idx += blockDim.x) {
      const unsigned long long j = idx % run;
      unsigned long long t = idx / run;
      const unsigned long long s = t % Sl;
      t /= Sl;
      const unsigned long long b = t % B;
      const int p = static_cast<int>(t / B);
      const unsigned long long off = src_offset(b, s, j, (c.rank - p + W) % W);
      mine[off] = in[off];
    }
  }
  bool ok = rank_barrier_block(c, ch, e + 1, PH_BARRIER_START);
  if (ok) {
    // Output enumerated as (p, b, s, j) with j in [0, run): nvec items in total.
    uint4* out = static_cast<uint4*>(a.out);
    for (unsigned long long idx = v0 + threadIdx.x; idx < v1; idx += blockDim.x) {
      const unsigned long long j = idx % run;
      unsigned long long t = idx / run;
      const unsigned long long s = t % Sl;
      t /= Sl;
      const unsigned long long b = t % B;
      const int p = static_cast<int>(t / B);
      const int src = (c.rank + p) % W;
      const unsigned long long src_off = src_offset(b, s, j, c.rank);
      // to_heads: out is [B, S, Hl, D]; otherwise in_p is [B, S, Hl, D] and out [B, Sl, H, D].
      const unsigned long long dst_off =
          a.a2a_to_heads ? ((b * (Sl * W) + src * Sl + s) * Hl) * dv + j
                         : ((b * Sl + s) * H + static_cast<unsigned long long>(src) * Hl) * dv + j;
      out[dst_off] = ld_sys_v4(static_cast<const uint4*>(a.sym[src]) + src_off);
    }
    ok = rank_barrier_block(c, ch, e + 2, PH_BARRIER_END);
  }
  end_epoch(c, ch, e + 2);
}

// ----------------------------------------------------------------- broadcast
// Root stages (copy_in) or already holds the data in sym[root]; everyone pulls.
// With a multicast alias the root pushes instead (one multimem.st per vector).
__global__ void __launch_bounds__(kCollThreads)
    bcast_kernel(const __grid_constant__ CollArgs args, const CollArgs* emu) {
  const CollArgs& a = pick_args(args, emu);
  const CbComm& c = a.comm;
  const uint32_t ch = cta_channel(0);
  const uint32_t e = begin_epoch(c, ch);
  const unsigned long long nvec = (a.nbytes + 15ull) / 16ull;
  unsigned long long v0, v1;
  slice_of(nvec, gridDim.x, blockIdx.x, &v0, &v1);
  const bool push = a.mc != nullptr;
  bool ok = true;
  if (push) {
    // Everyone must be done with the previous contents before the root overwrites them.
    ok = rank_barrier_block(c, ch, e + 1, PH_BARRIER_START);
    if (ok && c.rank == a.root) {
      const uint4* src = static_cast<const uint4*>(a.in);
      uint4* mc = static_cast<uint4*>(a.mc);
      const unsigned long long full = a.nbytes / 16ull;
      for (unsigned long long i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (i < full) {
          v = src[i];
        } else {
          unsigned char* d = reinterpret_cast<unsigned char*>(&v);
          const unsigned char* s = static_cast<const unsigned char*>(a.in) + i * 16ull;
          for (unsigned long long k = 0; k < a.nbytes - i * 16ull; ++k) d[k] = s[k];
        }
        mm_st_v4(mc + i, v);
      }
    }
    if (ok) ok = rank_barrier_block(c, ch, e + 2, PH_BARRIER_END);
    if (ok && a.copy_out) copy_bytes_slice(a.out, a.sym[c.rank], a.nbytes, v0, v1, false);
  } else {
    if (a.copy_in && c.rank == a.root)
      copy_bytes_slice(a.sym[c.rank], a.in, a.nbytes, v0, v1, true);
    ok = rank_barrier_block(c, ch, e + 1, PH_BARRIER_START);
    if (ok) {
      if (c.rank != a.root || a.out != a.in) {
        const uint4* sp = static_cast<const uint4*>(a.sym[a.root]);
        unsigned char* outb = static_cast<unsigned char*>(a.out);
        const unsigned long long full = a.nbytes / 16ull;
        for (unsigned long long i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
          const uint4 v = ld_sys_v4(sp + i);
          if (i < full) {
            reinterpret_cast<uint4*>(outb)[i] = v;
          } else {
            const unsigned char* s = reinterpret_cast<const unsigned char*>(&v);
            for (unsigned long long k = 0; k < a.nbytes - i * 16ull; ++k)
              outb[i * 16ull + k] = s[k];
          }
        }
      }
      ok = rank_barrier_block(c, ch, e + 2, PH_BARRIER_END);
    }
  }
  end_epoch(c, ch, e + 2);
}

// ------------------------------------------------------------------- barrier
// `iters` back-to-back barriers on channel 0 (iters > 1 is the latency benchmark
// of datasets/example017_intranode_gpu_barrier/nv/empty_intranode_gpu_barrier.cu:114-125).
__global__ void __launch_bounds__(32)
    barrier_kernel(const __grid_constant__ CollArgs args, const CollArgs* emu, int iters,
                   int use_nvls) {
  const CollArgs& a = pick_args(args, emu);
  const CbComm& c = a.comm;
  const uint32_t ch = cta_channel(0);
  if (use_nvls) {
    // The NVLS counter has its own running count kept in epoch[CHANNELS-1-ch].
    const uint32_t slot = CB_PAD_CHANNELS - 1 - ch;
    uint32_t e = begin_epoch(c, slot);
    bool ok = true;
    for (int i = 0; i < iters && ok; ++i) ok = nvls_barrier_block(c, ch, ++e);
    end_epoch(c, slot, e);
  } else {
    uint32_t e = begin_epoch(c, ch);
    bool ok = true;
    for (int i = 0; i < iters && ok; ++i) ok = rank_barrier_block(c, ch, e + 1 + i, 0);
    end_epoch(c, ch, e + iters);
  }
}

// ------------------------------------------------------------------ launcher
static int g_num_sms = 0;

template <typename K>
static cudaError_t launch_coll(K kernel, const CollArgs* args, const CollArgs* emu, int emu_world,
                               int blocks, int threads, cudaStream_t stream) {
  if (emu != nullptr) {
    // Emulated ranks wait on each other inside one grid: it must be co-resident.
    void* params[] = {const_cast<CollArgs*>(args), &emu};
    return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(blocks, emu_world),
                                       dim3(threads), params, 0, stream);
  }
  kernel<<<blocks, threads, 0, stream>>>(*args, nullptr);
  return cudaGetLastError();
}

}  // namespace cb

using namespace cb;

extern "C" {

enum CbCollOp : int {
  CB_OP_AR_ONESHOT = 0,
  CB_OP_AR_TWOSHOT = 1,
  CB_OP_AR_NVLS = 2,
  CB_OP_AG_PULL = 3,
  CB_OP_AG_PUSH = 4,
  CB_OP_RS = 5,
  CB_OP_A2A_FLAT = 6,
  CB_OP_A2A_4D = 7,
  CB_OP_BCAST = 8,
};

#define CB_DISPATCH_W(KERNEL_TMPL, ...)                                                   \
  switch (world) {                                                                        \
    case 1:                                                                               \
      err = launch_coll(KERNEL_TMPL<__VA_ARGS__ 1>, args, emu, emu_world, blocks, threads, st); \
      break;                                                                              \
    case 2:                                                                               \
      err = launch_coll(KERNEL_TMPL<__VA_ARGS__ 2>, args, emu, emu_world, blocks, threads, st); \
      break;                                                                              \
    case 4:                                                                               \
      err = launch_coll(KERNEL_TMPL<__VA_ARGS__ 4>, args, emu, emu_world, blocks, threads, st); \
      break;                                                                              \
    case 8:                                                                               \
      err = launch_coll(KERNEL_TMPL<__VA_ARGS__ 8>, args, emu, emu_world, blocks, threads, st); \
      break;                                                                              \
    default:                                                                              \
      return -3;                                                                          \
  }

#define CB_DISPATCH_DT_W(KERNEL_TMPL)                    \
  switch (args->dtype) {                                 \
    case CB_BF16:                                        \
      CB_DISPATCH_W(KERNEL_TMPL, CB_BF16, ) break;       \
    case CB_F16:                                         \
      CB_DISPATCH_W(KERNEL_TMPL, CB_F16, ) break;        \
    case CB_F32:                                         \
      CB_DISPATCH_W(KERNEL_TMPL, CB_F32, ) break;        \
    default:                                             \
      return -4;                                         \
  }

// Launches one collective.  `args` is this rank's argument block (host memory);
// `emu` (device memory, `emu_world` blocks) switches to single-GPU rank
// emulation.  Returns 0, or a negative code: -3 unsupported world size,
// -4 unsupported dtype, -5 unknown op, -1 launch error (see cb_last_cuda_error).
int cb_coll_launch(int op, const CollArgs* args, const CollArgs* emu, int emu_world, int blocks,
                   void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int world = args->comm.world;
  const int threads = kCollThreads;
  if (blocks < 1) blocks = 1;
  if (blocks > CB_PAD_CHANNELS / 2) blocks = CB_PAD_CHANNELS / 2;
  cudaError_t err = cudaSuccess;
  switch (op) {
    case CB_OP_AR_ONESHOT:
      CB_DISPATCH_DT_W(ar_oneshot_kernel);
      break;
    case CB_OP_AR_TWOSHOT:
      CB_DISPATCH_DT_W(ar_twoshot_kernel);
      break;
    case CB_OP_AR_NVLS:
      CB_DISPATCH_DT_W(ar_nvls_kernel);
      break;
    case CB_OP_AG_PULL:
      CB_DISPATCH_W(ag_pull_kernel, );
      break;
    case CB_OP_AG_PUSH:
      CB_DISPATCH_W(ag_push_kernel, );
      break;
    case CB_OP_RS:
      CB_DISPATCH_DT_W(rs_kernel);
      break;
    case CB_OP_A2A_FLAT:
      CB_DISPATCH_W(a2a_flat_kernel, );
      break;
    case CB_OP_A2A_4D:
      CB_DISPATCH_W(a2a_4d_kernel, );
      break;
    case CB_OP_BCAST:
      err = launch_coll(bcast_kernel, args, emu, emu_world, blocks, threads, st);
      break;
    default:
      return -5;
  }
  return err == cudaSuccess ? 0 : -1;
}

int cb_barrier_launch(const CollArgs* args, const CollArgs* emu, int emu_world, int iters,
                      int use_nvls, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t err;
  if (emu != nullptr) {
    void* params[] = {const_cast<CollArgs*>(args), &emu, &iters, &use_nvls};
    err = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(barrier_kernel), dim3(1, emu_world),
                                      dim3(32), params, 0, st);
  } else {
    barrier_kernel<<<1, 32, 0, st>>>(*args, nullptr, iters, use_nvls);
    err = cudaGetLastError();
  }
  return err == cudaSuccess ? 0 : -1;
}

int cb_sizeof_coll_args() { return static_cast<int>(sizeof(CollArgs)); }

}  // extern "C"
