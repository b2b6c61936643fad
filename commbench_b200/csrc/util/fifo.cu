// GPU <-> CPU queues.
//
//  * D2H trigger FIFO: device threads push 16-byte triggers {fst, snd}; a host
//    proxy thread polls and pops them.  Triggers live in mapped host memory, the
//    head ticket counter in device memory, the tail (consumed count) in mapped
//    host memory with a device-side cache.  Same roles as the MSCCL++-style FIFO
//    of datasets/example003_fifo_device2host/amd_nv/empty_fifo_test_unified.cu:431-494
//    (push/poll/sync on the device, poll/pop on the host, proxy thread :533-570).
//  * H2D task FIFO: the host pushes 8-byte tasks, a persistent kernel pops them
//    (datasets/example005_fifo_host2device/amd_nv/empty_h2dfifo_test_unified.cu:364-479).
//
// Every device-side wait is bounded: a push that finds the queue full for longer
// than the budget, or a consumer whose producer went away, records a status word
// and returns.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>
#include <time.h>

#include <atomic>
#include <string>
#include <thread>
#include <vector>

#include "../prim/ptx.cuh"

namespace cb {
void set_last_error(const std::string& s);

struct Trigger {
  unsigned long long fst;  // never 0 for a valid trigger
  unsigned long long snd;  // bit 63 is the "written" mark, flipped by push
};

struct D2HDevice {
  Trigger* triggers;              // mapped host memory (device alias)
  unsigned long long* head;       // device memory: next ticket
  unsigned long long* tail;       // mapped host memory (device alias): consumed count
  unsigned long long* tail_cache; // device memory
  int size;
};

// Returns the ticket (position) of the pushed trigger, or ~0 on time-out.
__device__ __forceinline__ unsigned long long d2h_push(const D2HDevice& f, unsigned long long fst,
                                                       unsigned long long snd,
                                                       unsigned long long timeout_ns,
                                                       uint32_t* status) {
  const unsigned long long ticket = atomicAdd(f.head, 1ull);
  // Wait for room: ticket < tail + size.  Check the cached tail first.
  if (ticket >= *reinterpret_cast<volatile unsigned long long*>(f.tail_cache) + f.size) {
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 0;; ++it) {
      const unsigned long long t = *reinterpret_cast<volatile unsigned long long*>(f.tail);
      if (ticket < t + f.size) {
        atomicMax(f.tail_cache, t);
        break;
      }
      if ((it & 15u) == 15u && globaltimer_ns() - t0 > timeout_ns) {
        report_status(status, CB_TIMEOUT_HOST_FLAG, 50, 0);
        return ~0ull;
      }
      __nanosleep(100);
    }
  }
  Trigger* slot = f.triggers + (ticket % f.size);
  // One 16-byte store; the host additionally checks the mark in `snd`.
  asm volatile("st.global.release.sys.v2.u64 [%0], {%1, %2};" ::"l"(slot), "l"(fst),
               "l"(snd ^ (1ull << 63))
               : "memory");
  return ticket;
}

// True once the trigger with this ticket has been consumed by the host.
__device__ __forceinline__ bool d2h_consumed(const D2HDevice& f, unsigned long long ticket) {
  return *reinterpret_cast<volatile unsigned long long*>(f.tail) > ticket;
}

__global__ void d2h_push_test_kernel(D2HDevice f, int per_thread, unsigned long long timeout_ns,
                                     uint32_t* status, unsigned long long* push_ns) {
  const unsigned long long gid = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
  for (int i = 0; i < per_thread; ++i) {
    const unsigned long long id = gid * per_thread + i + 1;  // non-zero
    const uint64_t t0 = globaltimer_ns();
    const unsigned long long tk = d2h_push(f, id, t0 & ~(1ull << 63), timeout_ns, status);
    if (tk == ~0ull) return;
    if (push_ns != nullptr && gid == 0 && i == 0) *push_ns = globaltimer_ns() - t0;
  }
}

struct D2HFifo {
  int size = 0;
  Trigger* triggers_h = nullptr;
  Trigger* triggers_d = nullptr;
  unsigned long long* head_d = nullptr;
  unsigned long long* tail_h = nullptr;
  unsigned long long* tail_d = nullptr;
  unsigned long long* tail_cache_d = nullptr;
  unsigned long long host_tail = 0;
  // proxy
  std::thread proxy;
  std::atomic<bool> stop{false};
  std::atomic<unsigned long long> popped{0};
  std::atomic<unsigned long long> checksum{0};
  std::atomic<unsigned long long> first_ns{0}, last_ns{0};
};

static unsigned long long host_now_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return static_cast<unsigned long long>(ts.tv_sec) * 1000000000ull + ts.tv_nsec;
}

static bool d2h_poll(D2HFifo* f, Trigger* out) {
  volatile Trigger* slot = f->triggers_h + (f->host_tail % f->size);
  const unsigned long long fst = slot->fst;
  if (fst == 0) return false;
  std::atomic_thread_fence(std::memory_order_acquire);
  const unsigned long long snd = slot->snd;
  if ((snd >> 63) == 0) return false;  // second half not visible yet
  out->fst = fst;
  out->snd = snd ^ (1ull << 63);
  return true;
}
static void d2h_pop(D2HFifo* f) {
  volatile Trigger* slot = f->triggers_h + (f->host_tail % f->size);
  slot->fst = 0;
  slot->snd = 0;
  std::atomic_thread_fence(std::memory_order_release);
  f->host_tail++;
  *reinterpret_cast<volatile unsigned long long*>(f->tail_h) = f->host_tail;
}

// ----------------------------------------------------------------- H2D FIFO
struct H2DDevice {
  const unsigned long long* items;  // mapped host memory (device alias), ring of `size`
  const unsigned long long* tail;   // mapped host: produced count (host writes)
  unsigned long long* head;         // mapped host: consumed count (device writes)
  int size;
};

// Persistent consumer: one thread pops `expect` items, writes each value and its
// pop time into `results[2*i], results[2*i+1]`.  Gives up (status) after `timeout_ns`
// without a new item.
__global__ void h2d_pop_kernel(H2DDevice f, unsigned long long expect, unsigned long long* results,
                               unsigned long long timeout_ns, uint32_t* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  unsigned long long head = *reinterpret_cast<volatile unsigned long long*>(f.head);
  for (unsigned long long i = 0; i < expect; ++i) {
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 0;; ++it) {
      if (*reinterpret_cast<const volatile unsigned long long*>(f.tail) > head) break;
      if ((it & 15u) == 15u && globaltimer_ns() - t0 > timeout_ns) {
        report_status(status, CB_TIMEOUT_HOST_FLAG, 51, static_cast<uint32_t>(i));
        return;
      }
    }
    __threadfence_system();
    const unsigned long long v =
        *reinterpret_cast<const volatile unsigned long long*>(f.items + (head % f.size));
    results[2 * i] = v;
    results[2 * i + 1] = globaltimer_ns();
    ++head;
    *reinterpret_cast<volatile unsigned long long*>(f.head) = head;
  }
}

struct H2DFifo {
  int size = 0;
  unsigned long long* items_h = nullptr;
  unsigned long long* items_d = nullptr;
  unsigned long long* ctl_h = nullptr;  // [0] tail, [8] head (separate cache lines)
  unsigned long long* ctl_d = nullptr;
  unsigned long long host_tail = 0;
};

}  // namespace cb

using namespace cb;

extern "C" {

int cb_d2h_fifo_create(int size, void** out) {
  if (size < 2 || size > (1 << 20)) {
    set_last_error("d2h fifo: size out of range");
    return -1;
  }
  D2HFifo* f = new D2HFifo();
  f->size = size;
  cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&f->triggers_h), sizeof(Trigger) * size,
                                cudaHostAllocMapped);
  if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&f->tail_h), 64, cudaHostAllocMapped);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&f->head_d), 16);
  if (e != cudaSuccess) {
    set_last_error(std::string("d2h fifo alloc: ") + cudaGetErrorString(e));
    delete f;
    return -1;
  }
  f->tail_cache_d = f->head_d + 1;
  memset(f->triggers_h, 0, sizeof(Trigger) * size);
  memset(f->tail_h, 0, 64);
  cudaMemset(f->head_d, 0, 16);
  cudaHostGetDevicePointer(reinterpret_cast<void**>(&f->triggers_d), f->triggers_h, 0);
  cudaHostGetDevicePointer(reinterpret_cast<void**>(&f->tail_d), f->tail_h, 0);
  *out = f;
  return 0;
}

// Host-side poll/pop for callers that run their own loop (returns 1 when a trigger was read).
int cb_d2h_fifo_poll(void* fifo, unsigned long long* fst, unsigned long long* snd) {
  Trigger t;
  if (!d2h_poll(static_cast<D2HFifo*>(fifo), &t)) return 0;
  *fst = t.fst;
  *snd = t.snd;
  return 1;
}
int cb_d2h_fifo_pop(void* fifo) {
  d2h_pop(static_cast<D2HFifo*>(fifo));
  return 0;
}

// Proxy thread: pops everything, counts, sums `fst`, remembers first/last arrival time.
int cb_d2h_fifo_proxy_start(void* fifo) {
  D2HFifo* f = static_cast<D2HFifo*>(fifo);
  f->stop = false;
  f->popped = 0;
  f->checksum = 0;
  f->first_ns = 0;
  f->last_ns = 0;
  f->proxy = std::thread([f] {
    Trigger t;
    while (!f->stop.load(std::memory_order_relaxed)) {
      if (d2h_poll(f, &t)) {
        const unsigned long long now = host_now_ns();
        if (f->popped.load() == 0) f->first_ns = now;
        f->last_ns = now;
        f->checksum += t.fst;
        d2h_pop(f);
        f->popped++;
      }
    }
  });
  return 0;
}
int cb_d2h_fifo_proxy_stop(void* fifo, unsigned long long* popped, unsigned long long* checksum,
                           unsigned long long* span_ns) {
  D2HFifo* f = static_cast<D2HFifo*>(fifo);
  f->stop = true;
  if (f->proxy.joinable()) f->proxy.join();
  *popped = f->popped;
  *checksum = f->checksum;
  *span_ns = f->last_ns.load() - f->first_ns.load();
  return 0;
}
unsigned long long cb_d2h_fifo_popped(void* fifo) { return static_cast<D2HFifo*>(fifo)->popped; }

int cb_d2h_fifo_push_test(void* fifo, int blocks, int threads, int per_thread,
                          unsigned long long timeout_ns, void* status, void* push_ns,
                          void* stream) {
  D2HFifo* f = static_cast<D2HFifo*>(fifo);
  D2HDevice d{f->triggers_d, f->head_d, f->tail_d, f->tail_cache_d, f->size};
  d2h_push_test_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      d, per_thread, timeout_ns, static_cast<uint32_t*>(status),
      static_cast<unsigned long long*>(push_ns));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int cb_d2h_fifo_destroy(void* fifo) {
  D2HFifo* f = static_cast<D2HFifo*>(fifo);
  if (f == nullptr) return 0;
  f->stop = true;
  if (f->proxy.joinable()) f->proxy.join();
  cudaFreeHost(f->triggers_h);
  cudaFreeHost(f->tail_h);
  cudaFree(f->head_d);
  delete f;
  return 0;
}

int cb_h2d_fifo_create(int size, void** out) {
  if (size < 2 || size > (1 << 20)) {
    set_last_error("h2d fifo: size out of range");
    return -1;
  }
  H2DFifo* f = new H2DFifo();
  f->size = size;
  cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&f->items_h), 8ull * size, cudaHostAllocMapped);
  if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&f->ctl_h), 256, cudaHostAllocMapped);
  if (e != cudaSuccess) {
    set_last_error(std::string("h2d fifo alloc: ") + cudaGetErrorString(e));
    delete f;
    return -1;
  }
  memset(f->items_h, 0, 8ull * size);
  memset(f->ctl_h, 0, 256);
  cudaHostGetDevicePointer(reinterpret_cast<void**>(&f->items_d), f->items_h, 0);
  cudaHostGetDevicePointer(reinterpret_cast<void**>(&f->ctl_d), f->ctl_h, 0);
  *out = f;
  return 0;
}

// Blocks while the ring is full; returns -2 if the consumer made no room within timeout_ms.
int cb_h2d_fifo_push(void* fifo, unsigned long long value, int timeout_ms) {
  H2DFifo* f = static_cast<H2DFifo*>(fifo);
  const unsigned long long t0 = host_now_ns();
  while (f->host_tail - *reinterpret_cast<volatile unsigned long long*>(f->ctl_h + 16) >=
         static_cast<unsigned long long>(f->size)) {
    if (host_now_ns() - t0 > static_cast<unsigned long long>(timeout_ms) * 1000000ull) {
      set_last_error("h2d fifo: full, consumer made no progress");
      return -2;
    }
  }
  f->items_h[f->host_tail % f->size] = value;
  std::atomic_thread_fence(std::memory_order_release);
  f->host_tail++;
  *reinterpret_cast<volatile unsigned long long*>(f->ctl_h) = f->host_tail;
  return 0;
}

int cb_h2d_fifo_launch_consumer(void* fifo, unsigned long long expect, void* results,
                                unsigned long long timeout_ns, void* status, void* stream) {
  H2DFifo* f = static_cast<H2DFifo*>(fifo);
  H2DDevice d{f->items_d, f->ctl_d, f->ctl_d + 16, f->size};
  h2d_pop_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      d, expect, static_cast<unsigned long long*>(results), timeout_ns,
      static_cast<uint32_t*>(status));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int cb_h2d_fifo_destroy(void* fifo) {
  H2DFifo* f = static_cast<H2DFifo*>(fifo);
  if (f == nullptr) return 0;
  cudaFreeHost(f->items_h);
  cudaFreeHost(f->ctl_h);
  delete f;
  return 0;
}

}  // extern "C"
