// Single-writer, multi-reader message queue in POSIX shared memory: the writer
// broadcasts byte messages (pickled objects on the Python side) to N readers on
// the same host.  A message that does not fit one slot travels in consecutive
// slots.  Every wait has a deadline.
//
// Same capability as the shared-memory MessageQueue of
// datasets/example100_vllm_shm_broadcast_object/nv/empty_vllm_shm_broadcast_object.py:94-135
// (writer rank 0, readers `dequeue(timeout)`), as a native ring buffer.
#include <errno.h>
#include <fcntl.h>
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <string>

namespace cb {
void set_last_error(const std::string& s);

static int64_t q_now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return int64_t(ts.tv_sec) * 1000 + ts.tv_nsec / 1000000;
}

struct QHeader {
  uint32_t magic;
  uint32_t n_readers;
  uint32_t nslots;
  uint32_t slot_bytes;
  std::atomic<uint64_t> written;          // slots published so far
  std::atomic<uint64_t> read_pos[16];     // slots consumed by each reader
};

struct SlotHeader {
  uint32_t nbytes;   // payload bytes in this slot
  uint32_t more;     // 1: the message continues in the next slot
};

struct ShmQueue {
  std::string name;
  int fd = -1;
  size_t map_bytes = 0;
  QHeader* h = nullptr;
  uint8_t* slots = nullptr;
  int reader = -1;  // -1: writer
  bool owner = false;
};

static size_t slot_stride(const QHeader* h) { return sizeof(SlotHeader) + h->slot_bytes; }

}  // namespace cb

using namespace cb;

extern "C" {

int cb_shmq_create(const char* name, int n_readers, int nslots, int slot_bytes, void** out) {
  if (n_readers < 1 || n_readers > 16 || nslots < 2 || slot_bytes < 64) {
    set_last_error("shmq: bad geometry (1..16 readers, >= 2 slots, >= 64-byte slots)");
    return -1;
  }
  ShmQueue* q = new ShmQueue();
  q->name = std::string("/") + name;
  q->owner = true;
  shm_unlink(q->name.c_str());
  q->fd = shm_open(q->name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  q->map_bytes = sizeof(QHeader) + size_t(nslots) * (sizeof(SlotHeader) + size_t(slot_bytes));
  if (q->fd < 0 || ftruncate(q->fd, off_t(q->map_bytes)) != 0) {
    set_last_error(std::string("shmq: shm_open/ftruncate: ") + strerror(errno));
    delete q;
    return -1;
  }
  void* p = mmap(nullptr, q->map_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, q->fd, 0);
  if (p == MAP_FAILED) {
    set_last_error(std::string("shmq: mmap: ") + strerror(errno));
    delete q;
    return -1;
  }
  q->h = static_cast<QHeader*>(p);
  q->h->n_readers = uint32_t(n_readers);
  q->h->nslots = uint32_t(nslots);
  q->h->slot_bytes = uint32_t(slot_bytes);
  q->h->written.store(0);
  for (int i = 0; i < 16; ++i) q->h->read_pos[i].store(0);
  std::atomic_thread_fence(std::memory_order_release);
  q->h->magic = 0x51554555u;
  q->slots = reinterpret_cast<uint8_t*>(q->h + 1);
  *out = q;
  return 0;
}

int cb_shmq_open(const char* name, int reader, int timeout_ms, void** out) {
  ShmQueue* q = new ShmQueue();
  q->name = std::string("/") + name;
  q->reader = reader;
  const int64_t deadline = q_now_ms() + timeout_ms;
  for (;;) {
    q->fd = shm_open(q->name.c_str(), O_RDWR, 0600);
    if (q->fd >= 0) {
      struct stat st;
      if (fstat(q->fd, &st) == 0 && size_t(st.st_size) >= sizeof(QHeader)) {
        q->map_bytes = size_t(st.st_size);
        break;
      }
      close(q->fd);
      q->fd = -1;
    }
    if (q_now_ms() > deadline) {
      set_last_error("shmq: timed out waiting for the writer to create the queue");
      delete q;
      return -2;
    }
    usleep(500);
  }
  void* p = mmap(nullptr, q->map_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, q->fd, 0);
  if (p == MAP_FAILED) {
    set_last_error(std::string("shmq: mmap: ") + strerror(errno));
    delete q;
    return -1;
  }
  q->h = static_cast<QHeader*>(p);
  while (*reinterpret_cast<volatile uint32_t*>(&q->h->magic) != 0x51554555u) {
    if (q_now_ms() > deadline) {
      set_last_error("shmq: queue never became ready");
      munmap(p, q->map_bytes);
      delete q;
      return -2;
    }
    usleep(200);
  }
  if (reader < 0 || uint32_t(reader) >= q->h->n_readers) {
    set_last_error("shmq: reader index out of range");
    munmap(p, q->map_bytes);
    delete q;
    return -1;
  }
  q->slots = reinterpret_cast<uint8_t*>(q->h + 1);
  *out = q;
  return 0;
}

// Writer: publishes one message (any size).  -2 when a reader stalls past the deadline.
int cb_shmq_write(void* queue, const void* data, long long nbytes, int timeout_ms) {
  ShmQueue* q = static_cast<ShmQueue*>(queue);
  QHeader* h = q->h;
  const int64_t deadline = q_now_ms() + timeout_ms;
  const uint8_t* src = static_cast<const uint8_t*>(data);
  long long left = nbytes;
  do {
    const uint64_t w = h->written.load(std::memory_order_relaxed);
    // The slot is free once every reader has consumed slot w - nslots.
    for (uint32_t spins = 0;; ++spins) {
      uint64_t slowest = ~0ull;
      for (uint32_t r = 0; r < h->n_readers; ++r) {
        const uint64_t rp = h->read_pos[r].load(std::memory_order_acquire);
        if (rp < slowest) slowest = rp;
      }
      if (w - slowest < h->nslots) break;
      if ((spins & 255u) == 255u) {
        if (q_now_ms() > deadline) {
          set_last_error("shmq: a reader did not drain the queue in time");
          return -2;
        }
        usleep(50);
      }
    }
    uint8_t* slot = q->slots + (w % h->nslots) * slot_stride(h);
    SlotHeader* sh = reinterpret_cast<SlotHeader*>(slot);
    const uint32_t n = uint32_t(left < (long long)h->slot_bytes ? left : h->slot_bytes);
    memcpy(slot + sizeof(SlotHeader), src, n);
    sh->nbytes = n;
    src += n;
    left -= n;
    sh->more = left > 0 ? 1u : 0u;
    h->written.store(w + 1, std::memory_order_release);
  } while (left > 0);
  return 0;
}

// Reader: receives one message into `buf` (capacity `cap`).  Returns 0 and the size,
// -2 on time-out (nothing consumed beyond complete slots already read), -3 if `cap` is short.
int cb_shmq_read(void* queue, void* buf, long long cap, long long* nbytes, int timeout_ms) {
  ShmQueue* q = static_cast<ShmQueue*>(queue);
  QHeader* h = q->h;
  const int64_t deadline = q_now_ms() + timeout_ms;
  uint8_t* dst = static_cast<uint8_t*>(buf);
  long long got = 0;
  for (;;) {
    const uint64_t rp = h->read_pos[q->reader].load(std::memory_order_relaxed);
    for (uint32_t spins = 0; h->written.load(std::memory_order_acquire) <= rp; ++spins) {
      if ((spins & 255u) == 255u) {
        if (q_now_ms() > deadline) {
          set_last_error("shmq: no message within the deadline");
          return -2;
        }
        usleep(20);
      }
    }
    const uint8_t* slot = q->slots + (rp % h->nslots) * slot_stride(h);
    const SlotHeader* sh = reinterpret_cast<const SlotHeader*>(slot);
    const uint32_t n = sh->nbytes;
    const uint32_t more = sh->more;
    if (got + n > cap) {
      set_last_error("shmq: receive buffer too small");
      return -3;
    }
    memcpy(dst + got, slot + sizeof(SlotHeader), n);
    got += n;
    h->read_pos[q->reader].store(rp + 1, std::memory_order_release);
    if (!more) break;
  }
  *nbytes = got;
  return 0;
}

int cb_shmq_close(void* queue) {
  ShmQueue* q = static_cast<ShmQueue*>(queue);
  if (q == nullptr) return 0;
  if (q->h) munmap(q->h, q->map_bytes);
  if (q->fd >= 0) close(q->fd);
  if (q->owner) shm_unlink(q->name.c_str());
  delete q;
  return 0;
}

}  // extern "C"
