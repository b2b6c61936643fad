// GPU utility probes: copy bandwidth at 4/8/16-byte vector widths (local HBM,
// peer memory, mapped host memory), remote-store patterns with a flag per chunk,
// flag ping-pong latency between two GPUs, %globaltimer / nanosleep accuracy,
// mbarrier round-trip inside a CTA, TMA bulk gmem->smem streaming, device
// attributes.  Their results feed the roofline constants of the harness.
//
// Reference counterparts (one program each there, one entry point each here):
//   datasets/example077_GPU_vectorized_copy_widths/nv/empty_vectorized_copy_widths.cu:28,149
//   datasets/example074_GPU_p2p_d2d_bandwidth/nv/empty_p2p_d2d_bandwidth.cu:29-36,178-186
//   datasets/example075_GPU_d2h_copy_bandwidth/nv/empty_d2h_copy_bandwidth.cu:29,157
//   datasets/example073_GPU_p2p_pingpong_latency/nv/empty_p2p_pingpong_latency.cu:30-56
//   datasets/example076_GPU_globaltimer_nanosleep/nv/empty_globaltimer_nanosleep.cu:25-36
//   datasets/example072_GPU_barrier_within_CTA/nv/empty_gpu_barrier_within_cta.cu:44-84
//   datasets/example094_TMA_bulk_copy_gmem_to_smem/nv/empty_tma_bulk_copy.cu:28-97
//   datasets/example010_list_gpu_attributes/nv/empty_list_gpu_attributes.cpp:17-52
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <string>

#include "../prim/mbarrier.cuh"
#include "../prim/multimem.cuh"
#include "../prim/tma.cuh"

namespace cb {
void set_last_error(const std::string& s);

// ------------------------------------------------------------ vector-width copy
template <typename V>
__global__ void copy_width_kernel(V* __restrict__ dst, const V* __restrict__ src, size_t n) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (; i < n; i += stride) dst[i] = src[i];
}

// ------------------------------------------------------- remote-store patterns
// Each warp owns a contiguous slice and writes it 512 bytes per instruction.
// mode & 15 = 0: st.global.v4 (weak)   1: st.relaxed.sys.v4   2: multimem.st.v4
// After every `fence_every` instructions (0 = only at the end) the warp runs a
// system-scope fence (sequentially consistent = __threadfence_system() by default,
// fence.acq_rel.sys when mode & 16) and lane 0 adds 1 to `flag`: the cost of
// "data, then flag" at that granularity.
__global__ void store_pattern_kernel(uint4* dst, const uint4* __restrict__ src, size_t nvec,
                                     int mode, int fence_every, uint32_t* flag) {
  const size_t warps = static_cast<size_t>(gridDim.x) * (blockDim.x >> 5);
  const size_t warp = blockIdx.x * static_cast<size_t>(blockDim.x >> 5) + (threadIdx.x >> 5);
  const size_t per = (nvec / 32 + warps - 1) / warps * 32;  // vectors per warp, multiple of 32
  size_t b = warp * per, e = b + per;
  if (e > nvec) e = nvec;
  const uint32_t lane = threadIdx.x & 31u;
  int since = 0;
  const bool acq_rel = (mode & 16) != 0;
  mode &= 15;
  for (size_t i = b + lane; i < e; i += 32) {
    const uint4 v = src[i];
    if (mode == 0) {
      dst[i] = v;
    } else if (mode == 1) {
      st_sys_v4(dst + i, v);
    } else {
      mm_st_v4(dst + i, v);
    }
    if (fence_every > 0 && ++since == fence_every) {
      since = 0;
      if (acq_rel) fence_acq_rel_sys(); else __threadfence_system();
      __syncwarp();
      if (lane == 0 && flag != nullptr) red_relaxed_sys_add(flag, 1u);
    }
  }
  __threadfence_system();
  __syncwarp();
  if (lane == 0 && flag != nullptr) red_release_sys_add(flag, 1u);
}

// --------------------------------------------------------------- ping-pong
// Two GPUs, one warp each.  `mine` is local, `theirs` is the peer's word.
// Rank 0 writes i+1 and waits for the echo; rank 1 waits and echoes.
__global__ void pingpong_kernel(uint32_t* mine, uint32_t* theirs, int rank, int rounds,
                                uint32_t base, unsigned long long timeout_ns, uint32_t* status,
                                unsigned long long* elapsed_ns) {
  if (threadIdx.x != 0) return;
  const uint64_t t0 = globaltimer_ns();
  for (int i = 0; i < rounds; ++i) {
    const uint32_t v = base + static_cast<uint32_t>(i) + 1u;
    if (rank == 0) {
      st_release_sys(theirs, v);
      if (!wait_flag_ge_sys(mine, v, timeout_ns, status, 40, i)) break;
    } else {
      if (!wait_flag_ge_sys(mine, v, timeout_ns, status, 40, i)) break;
      st_release_sys(theirs, v);
    }
  }
  *elapsed_ns = globaltimer_ns() - t0;
}

// ------------------------------------------------------ globaltimer / nanosleep
__global__ void nanosleep_probe_kernel(unsigned request_ns, int reps, unsigned long long* out) {
  if (threadIdx.x != 0) return;
  unsigned long long total = 0;
  for (int i = 0; i < reps; ++i) {
    const uint64_t t0 = globaltimer_ns();
    __nanosleep(request_ns);
    total += globaltimer_ns() - t0;
  }
  out[0] = total / (reps > 0 ? reps : 1);
  // timer resolution: smallest non-zero step seen in a tight loop
  uint64_t prev = globaltimer_ns(), best = ~0ull;
  for (int i = 0; i < 4096; ++i) {
    const uint64_t now = globaltimer_ns();
    if (now != prev && now - prev < best) best = now - prev;
    prev = now;
  }
  out[1] = best;
}

// ------------------------------------------------------ mbarrier inside a CTA
// Warp 0 is the producer, every other thread a consumer: `iters` rounds of
// arrive / try_wait on two mbarriers (ready, consumed).
__global__ void mbarrier_bench_kernel(int iters, unsigned long long* cycles, uint32_t* status) {
  __shared__ uint64_t ready, consumed;
  const uint32_t consumers = blockDim.x > 32 ? blockDim.x - 32 : 0;
  if (threadIdx.x == 0) {
    mbar_init(&ready, 1);
    mbar_init(&consumed, consumers > 0 ? consumers : 1);
    fence_mbar_init();
  }
  __syncthreads();
  const long long t0 = clock64();
  bool ok = true;
  for (int i = 0; i < iters && ok; ++i) {
    const uint32_t par = static_cast<uint32_t>(i) & 1u;
    if (threadIdx.x == 0) {
      mbar_arrive(&ready);
      if (consumers > 0) ok = mbar_wait(&consumed, par, nullptr, status, 0x600);
      else mbar_arrive(&consumed);
    } else if (threadIdx.x >= 32) {
      ok = mbar_wait(&ready, par, nullptr, status, 0x601);
      mbar_arrive(&consumed);
    }
  }
  if (threadIdx.x == 0) cycles[0] = static_cast<unsigned long long>(clock64() - t0);
}

// ------------------------------------------------- TMA bulk gmem -> smem stream
// Every CTA streams `iters` tiles of `tile_bytes` through a `stages`-deep ring of
// shared-memory buffers (one producer thread; consumers only acknowledge).
__global__ void tma_stream_kernel(const uint8_t* __restrict__ src, size_t src_bytes,
                                  uint32_t tile_bytes, int stages, int iters,
                                  unsigned long long* sink, uint32_t* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full[8];
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  const size_t ntiles = src_bytes / tile_bytes;
  size_t t = (static_cast<size_t>(blockIdx.x) * 977) % ntiles;
  unsigned long long acc = 0;
  for (int i = 0; i < stages && i < iters; ++i) {
    mbar_arrive_expect_tx(&full[i], tile_bytes);
    bulk_load_1d(smem + static_cast<size_t>(i) * tile_bytes, src + t * tile_bytes, tile_bytes,
                 &full[i]);
    t = (t + gridDim.x) % ntiles;
  }
  for (int i = 0; i < iters; ++i) {
    const int s = i % stages;
    if (!mbar_wait(&full[s], (static_cast<uint32_t>(i / stages)) & 1u, nullptr, status, 0x700 + s))
      break;
    acc += *reinterpret_cast<volatile unsigned long long*>(smem + static_cast<size_t>(s) * tile_bytes);
    if (i + stages < iters) {
      mbar_arrive_expect_tx(&full[s], tile_bytes);
      bulk_load_1d(smem + static_cast<size_t>(s) * tile_bytes, src + t * tile_bytes, tile_bytes,
                   &full[s]);
      t = (t + gridDim.x) % ntiles;
    }
  }
  sink[blockIdx.x] = acc;
}

}  // namespace cb

using namespace cb;

// mean(|x|) of a bf16 tensor in one pass (the metric the flagship step reads back): 16-byte
// loads, fp32 partial sums per thread, warp shuffles, one atomicAdd per block; the last block
// to finish writes sum / n and re-arms the two scratch words for the next call.
__global__ void __launch_bounds__(256)
    abs_mean_bf16_kernel(const uint4* __restrict__ x, long long nvec, long long n, float* out,
                         float* scratch_sum, unsigned int* scratch_count) {
  float acc = 0.f;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < nvec; i += 256ll * gridDim.x) {
    const uint4 v = x[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      acc += fabsf(f.x) + fabsf(f.y);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float warp_sum[8];
  __shared__ bool last;
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float b = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) b += warp_sum[w];
    atomicAdd(scratch_sum, b);
    __threadfence();
    last = atomicAdd(scratch_count, 1u) == gridDim.x - 1;
    if (last) {
      __threadfence();
      const float total = atomicExch(scratch_sum, 0.f);
      *out = total / static_cast<float>(n);
      *scratch_count = 0u;
    }
  }
}

extern "C" {

// width in {4, 8, 16} bytes.  dst may be local, peer-mapped or mapped host memory.
int cb_probe_copy(void* dst, const void* src, long long bytes, int width, int blocks, int threads,
                  void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (blocks < 1 || threads < 32 || threads > 1024) return -1;
  switch (width) {
    case 4:
      copy_width_kernel<uint32_t><<<blocks, threads, 0, st>>>(
          static_cast<uint32_t*>(dst), static_cast<const uint32_t*>(src), size_t(bytes) / 4);
      break;
    case 8:
      copy_width_kernel<uint2><<<blocks, threads, 0, st>>>(
          static_cast<uint2*>(dst), static_cast<const uint2*>(src), size_t(bytes) / 8);
      break;
    case 16:
      copy_width_kernel<uint4><<<blocks, threads, 0, st>>>(
          static_cast<uint4*>(dst), static_cast<const uint4*>(src), size_t(bytes) / 16);
      break;
    default:
      set_last_error("cb_probe_copy: width must be 4, 8 or 16");
      return -1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int cb_probe_store_pattern(void* dst, const void* src, long long bytes, int mode, int fence_every,
                           void* flag, int blocks, int threads, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  store_pattern_kernel<<<blocks, threads, 0, st>>>(static_cast<uint4*>(dst),
                                                   static_cast<const uint4*>(src),
                                                   size_t(bytes) / 16, mode, fence_every,
                                                   static_cast<uint32_t*>(flag));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int cb_probe_pingpong(void* mine, void* theirs, int rank, int rounds, unsigned base,
                      unsigned long long timeout_ns, void* status, void* elapsed_ns,
                      void* stream) {
  pingpong_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint32_t*>(mine), static_cast<uint32_t*>(theirs), rank, rounds, base, timeout_ns,
      static_cast<uint32_t*>(status), static_cast<unsigned long long*>(elapsed_ns));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int cb_probe_nanosleep(unsigned request_ns, int reps, void* out2, void* stream) {
  nanosleep_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      request_ns, reps, static_cast<unsigned long long*>(out2));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int cb_probe_mbarrier(int threads, int iters, void* cycles, void* status, void* stream) {
  if (threads < 32 || threads > 1024) return -1;
  mbarrier_bench_kernel<<<1, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      iters, static_cast<unsigned long long*>(cycles), static_cast<uint32_t*>(status));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int cb_probe_tma_stream(const void* src, long long src_bytes, int tile_bytes, int stages, int iters,
                        int blocks, void* sink, void* status, void* stream) {
  if (stages < 1 || stages > 8 || tile_bytes % 16 != 0 || tile_bytes * stages > 200 * 1024) {
    set_last_error("cb_probe_tma_stream: 1..8 stages, tile multiple of 16 B, ring <= 200 KB");
    return -1;
  }
  const int smem = tile_bytes * stages;
  cudaError_t e = cudaFuncSetAttribute(tma_stream_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return -1;
  tma_stream_kernel<<<blocks, 32, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), size_t(src_bytes), uint32_t(tile_bytes), stages, iters,
      static_cast<unsigned long long*>(sink), static_cast<uint32_t*>(status));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Device attributes as one JSON object written into `buf` (returns its length, or -1).
int cb_probe_attributes_json(int device, char* buf, int buflen) {
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, device) != cudaSuccess) {
    set_last_error("cudaGetDeviceProperties failed");
    (void)cudaGetLastError();
    return -1;
  }
  int clk = 0, mclk = 0, coop = 0;
  cudaDeviceGetAttribute(&clk, cudaDevAttrClockRate, device);
  cudaDeviceGetAttribute(&mclk, cudaDevAttrMemoryClockRate, device);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device);
  int n = snprintf(
      buf, size_t(buflen),
      "{\"name\": \"%s\", \"compute_capability\": \"%d.%d\", \"sm_count\": %d, "
      "\"global_mem_bytes\": %llu, \"l2_bytes\": %d, \"smem_per_block_optin\": %llu, "
      "\"smem_per_sm\": %llu, \"regs_per_sm\": %d, \"max_threads_per_sm\": %d, "
      "\"warp_size\": %d, \"sm_clock_khz\": %d, \"mem_clock_khz\": %d, \"mem_bus_bits\": %d, "
      "\"cooperative_launch\": %d, \"unified_addressing\": %d, \"can_map_host\": %d, "
      "\"ecc\": %d, \"pci\": \"%04x:%02x:%02x\"}",
      p.name, p.major, p.minor, p.multiProcessorCount, (unsigned long long)p.totalGlobalMem,
      p.l2CacheSize, (unsigned long long)p.sharedMemPerBlockOptin,
      (unsigned long long)p.sharedMemPerMultiprocessor, p.regsPerMultiprocessor,
      p.maxThreadsPerMultiProcessor, p.warpSize, clk, mclk, p.memoryBusWidth, coop,
      p.unifiedAddressing, p.canMapHostMemory, p.ECCEnabled, p.pciDomainID, p.pciBusID,
      p.pciDeviceID);
  return n < buflen ? n : -1;
}


// out[0] = mean(|x[0..n)|) for bf16 x (16-byte aligned, n % 8 == 0).  `scratch` = two zeroed
// 4-byte words that the kernel leaves zeroed.  One launch.
int cb_abs_mean_bf16(const void* x, long long n, float* out, void* scratch, void* stream) {
  if (n <= 0 || (n % 8) != 0 || (reinterpret_cast<uintptr_t>(x) & 15u) != 0 || out == nullptr ||
      scratch == nullptr) {
    set_last_error("cb_abs_mean_bf16: n > 0, n % 8 == 0, 16-byte aligned input, out and scratch");
    return -1;
  }
  const long long nvec = n / 8;
  long long blocks = (nvec + 255) / 256;
  if (blocks > 592) blocks = 592;
  abs_mean_bf16_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), nvec, n, out, static_cast<float*>(scratch),
      static_cast<unsigned int*>(scratch) + 1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(std::string("abs_mean launch: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // extern "C"
