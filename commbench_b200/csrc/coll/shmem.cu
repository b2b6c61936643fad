// One-sided primitives on the symmetric heap, the operations the reference reaches through
// NVSHMEM and MSCCL++ memory channels, written as plain kernels over peer pointers:
//   put + signal   (nvshmemx_putmem_nbi_block + quiet + signal_op / MemoryChannel::put + signal)
//                  datasets/example033_nvshmem_put_and_signal/nv/empty_nvshmem_put_and_signal.cu:33-84
//                  datasets/example038_mscclpp_mc_put_easy/empty_mscclpp_memorychannel_put_easy.cu:163-173
//   wait + get     (signal / wait / MemoryChannel::get)
//                  datasets/example039_mscclpp_mc_get_easy/empty_mscclpp_memorychannel_get_easy.cu:158-168
//   atomic fetch-inc on one PE's counter
//                  datasets/example032_nvshmem_atomic_fetch_inc/nv/empty_nvshmem_atomic_fetch_inc.cu:54-63
//   tile put with a flag per tile, consumer waits per tile
//                  datasets/example035_nvshmem_tiled_produce_consume/nv/
//                  empty_nvshmem_tiled_produce_consume.cu:110-132
// Every wait is bounded and reports a status word.
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../prim/barrier.cuh"

namespace cb {
void set_last_error(const std::string& s);

enum : uint32_t { PH_SHMEM_WAIT = 60, PH_SHMEM_TILE = 61 };

// Copy `nvec` 16-byte vectors to `dst` (peer memory); the last CTA to finish releases
// and then sets / adds the signal word at the destination.
__global__ void __launch_bounds__(512)
    put_signal_kernel(uint4* dst, const uint4* __restrict__ src, unsigned long long nvec,
                      uint32_t* signal, uint32_t value, int add, uint32_t* done_ctas) {
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
  unsigned long long i = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    st_sys_v4(dst + i, a);
    st_sys_v4(dst + i + stride, b);
    st_sys_v4(dst + i + 2 * stride, c);
    st_sys_v4(dst + i + 3 * stride, d);
  }
  for (; i < nvec; i += stride) st_sys_v4(dst + i, src[i]);
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();  // this CTA's stores precede the counter bump
    if (atomicAdd(done_ctas, 1u) == gridDim.x - 1) {
      *done_ctas = 0u;
      fence_acq_rel_sys();
      if (signal != nullptr) {
        if (add) red_relaxed_sys_add(signal, value);
        else st_relaxed_sys(signal, value);
      }
    }
  }
}

// Wait until *signal >= value, then (optionally) pull `nvec` vectors from `src` (peer memory).
__global__ void __launch_bounds__(512)
    wait_get_kernel(uint4* dst, const uint4* src, unsigned long long nvec, const uint32_t* signal,
                    uint32_t value, unsigned long long timeout_ns, uint32_t* status) {
  bool ok = true;
  if (signal != nullptr && threadIdx.x == 0)
    ok = wait_flag_ge_sys(signal, value, timeout_ns, status, PH_SHMEM_WAIT, blockIdx.x);
  if (__syncthreads_and(ok ? 1 : 0) == 0) return;
  if (dst == nullptr) return;
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
  unsigned long long i = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    const uint4 a = ld_sys_v4(src + i), b = ld_sys_v4(src + i + stride),
                c = ld_sys_v4(src + i + 2 * stride), d = ld_sys_v4(src + i + 3 * stride);
    dst[i] = a;
    dst[i + stride] = b;
    dst[i + 2 * stride] = c;
    dst[i + 3 * stride] = d;
  }
  for (; i < nvec; i += stride) dst[i] = ld_sys_v4(src + i);
}

// `n` fetch-and-increments on a counter that lives on one PE; tickets[i] = value fetched.
__global__ void atomic_fetch_inc_kernel(unsigned long long* counter, int n,
                                        unsigned long long* tickets, unsigned long long* cycles) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const long long t0 = clock64();
  for (int i = 0; i < n; ++i)
    tickets[i] = atom_add_relaxed_sys_u64(reinterpret_cast<uint64_t*>(counter), 1ull);
  *cycles = static_cast<unsigned long long>(clock64() - t0);
}

// Producer: CTA t copies tile t (TS x TS floats out of a side x side matrix) into the peer's
// matrix, releases, raises flag[t] at the peer.
__global__ void __launch_bounds__(256)
    tile_put_kernel(float* dst, const float* __restrict__ src, int side, int ts, uint32_t* flags,
                    uint32_t value) {
  const int tiles_per_row = side / ts;
  const int t = blockIdx.x;
  const int r0 = (t / tiles_per_row) * ts, c0 = (t % tiles_per_row) * ts;
  for (int i = threadIdx.x; i < ts * ts; i += blockDim.x) {
    const int r = r0 + i / ts, c = c0 + i % ts;
    asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(dst + static_cast<size_t>(r) * side + c),
                 "f"(src[static_cast<size_t>(r) * side + c])
                 : "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    st_relaxed_sys(flags + t, value);
  }
}

// Consumer: CTA t waits for flag[t], then sums its tile into partial[t].
__global__ void __launch_bounds__(256)
    tile_consume_kernel(const float* m, int side, int ts, const uint32_t* flags, uint32_t value,
                        float* partial, unsigned long long timeout_ns, uint32_t* status) {
  const int tiles_per_row = side / ts;
  const int t = blockIdx.x;
  bool ok = true;
  if (threadIdx.x == 0)
    ok = wait_flag_ge_sys(flags + t, value, timeout_ns, status, PH_SHMEM_TILE, t);
  if (__syncthreads_and(ok ? 1 : 0) == 0) return;
  const int r0 = (t / tiles_per_row) * ts, c0 = (t % tiles_per_row) * ts;
  float s = 0.f;
  for (int i = threadIdx.x; i < ts * ts; i += blockDim.x)
    s += __ldcg(m + static_cast<size_t>(r0 + i / ts) * side + c0 + i % ts);
  __shared__ float red[8];
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) tot += red[w];
    partial[t] = tot;
  }
}

}  // namespace cb

using namespace cb;

extern "C" {

// `done_ctas`: one zeroed uint32 of local device memory (scratch of the last-CTA pattern).
int cb_shmem_put_signal(void* dst, const void* src, long long nbytes, void* signal, unsigned value,
                        int add, void* done_ctas, int blocks, void* stream) {
  if (nbytes % 16 != 0 || blocks < 1) {
    set_last_error("shmem put: size must be a multiple of 16 bytes");
    return -1;
  }
  put_signal_kernel<<<blocks, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(dst), static_cast<const uint4*>(src),
      static_cast<unsigned long long>(nbytes / 16), static_cast<uint32_t*>(signal), value, add,
      static_cast<uint32_t*>(done_ctas));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// dst == nullptr: wait only.
int cb_shmem_wait_get(void* dst, const void* src, long long nbytes, const void* signal,
                      unsigned value, unsigned long long timeout_ns, void* status, int blocks,
                      void* stream) {
  if (nbytes % 16 != 0 || blocks < 1) {
    set_last_error("shmem get: size must be a multiple of 16 bytes");
    return -1;
  }
  wait_get_kernel<<<blocks, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(dst), static_cast<const uint4*>(src),
      static_cast<unsigned long long>(nbytes / 16), static_cast<const uint32_t*>(signal), value,
      timeout_ns, static_cast<uint32_t*>(status));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int cb_shmem_atomic_fetch_inc(void* counter, int n, void* tickets, void* cycles, void* stream) {
  atomic_fetch_inc_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned long long*>(counter), n, static_cast<unsigned long long*>(tickets),
      static_cast<unsigned long long*>(cycles));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int cb_shmem_tile_put(void* dst, const void* src, int side, int ts, void* flags, unsigned value,
                      void* stream) {
  if (ts < 1 || side % ts != 0) {
    set_last_error("tile put: side must be a multiple of the tile size");
    return -1;
  }
  const int tiles = (side / ts) * (side / ts);
  tile_put_kernel<<<tiles, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<float*>(dst), static_cast<const float*>(src), side, ts,
      static_cast<uint32_t*>(flags), value);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int cb_shmem_tile_consume(const void* m, int side, int ts, const void* flags, unsigned value,
                          void* partial, unsigned long long timeout_ns, void* status,
                          void* stream) {
  if (ts < 1 || side % ts != 0) return -1;
  const int tiles = (side / ts) * (side / ts);
  tile_consume_kernel<<<tiles, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(m), side, ts, static_cast<const uint32_t*>(flags), value,
      static_cast<float*>(partial), timeout_ns, static_cast<uint32_t*>(status));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
