// Rendezvous between the rank processes of one host: file descriptors travel
// over abstract unix sockets (SCM_RIGHTS), a POSIX shared-memory mailbox gives a
// host barrier and small all-gathers.  Every wait has a deadline.
//
// Capability parity: the KittensBroker of the reference's ThunderKittens
// examples (sync / exchange_fds / broadcast_fd:
// datasets/example060_thunderkitten_all_reduce_hard/nv/
// empty_thunderkitten_all_reduce.cu:112-146) and the unix-socket handle shipping
// of datasets/example012_gpu_ipc_comm_with_NVLink/nv/empty_gpu_ipc_comm.cu:43-79.
// Nothing here touches CUDA, so it is tested on a CPU-only machine with memfd
// descriptors standing in for exported GPU allocations.
#include <errno.h>
#include <fcntl.h>
#include <poll.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <map>
#include <string>
#include <vector>

#include "../prim/status.h"

namespace cb {
void set_last_error(const std::string& s);

static int64_t now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return int64_t(ts.tv_sec) * 1000 + ts.tv_nsec / 1000000;
}

struct Mailbox {  // lives in POSIX shared memory, one per job
  std::atomic<uint32_t> arrive[2];  // sense-reversing barrier counters
  std::atomic<uint32_t> ready;
  uint8_t slots[CB_MAX_RANKS][256];  // small all-gather payloads
};

struct Broker {
  std::string name;
  int rank = 0, world = 1;
  int listen_fd = -1;
  int shm_fd = -1;
  Mailbox* mb = nullptr;
  uint32_t barrier_round = 0;
  uint32_t fd_round = 0;
  // descriptors that arrived for a later round than the one being collected
  std::map<std::pair<uint32_t, int>, int> pending;
};

static void make_addr(const std::string& name, int rank, sockaddr_un* a, socklen_t* len) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  // Abstract namespace: leading NUL, vanishes with the process, nothing to unlink.
  std::string path = name + "." + std::to_string(rank);
  size_t n = path.size() < sizeof(a->sun_path) - 2 ? path.size() : sizeof(a->sun_path) - 2;
  memcpy(a->sun_path + 1, path.data(), n);
  *len = socklen_t(offsetof(sockaddr_un, sun_path) + 1 + n);
}

struct FdMsg {
  uint32_t round;
  int32_t src;
};

static int send_fd(int sock, const FdMsg& m, int fd) {
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  iovec iov;
  iov.iov_base = const_cast<FdMsg*>(&m);
  iov.iov_len = sizeof(m);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  return sendmsg(sock, &msg, 0) == ssize_t(sizeof(m)) ? 0 : -1;
}

static int recv_fd(int sock, FdMsg* m, int* fd) {
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  iovec iov;
  iov.iov_base = m;
  iov.iov_len = sizeof(*m);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  if (recvmsg(sock, &msg, 0) != ssize_t(sizeof(*m))) return -1;
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (c == nullptr || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) return -1;
  memcpy(fd, CMSG_DATA(c), sizeof(int));
  return 0;
}

}  // namespace cb

using namespace cb;

extern "C" {

// `name` is a job-unique string every rank agrees on (the Python layer derives
// it from the torch.distributed store).  Rank 0 creates the mailbox.
int cb_broker_create(const char* name, int rank, int world, int timeout_ms, void** out) {
  if (world < 1 || world > CB_MAX_RANKS || rank < 0 || rank >= world) {
    set_last_error("broker: bad rank/world");
    return -1;
  }
  Broker* b = new Broker();
  b->name = name;
  b->rank = rank;
  b->world = world;
  b->listen_fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (b->listen_fd < 0) {
    set_last_error(std::string("broker: socket: ") + strerror(errno));
    delete b;
    return -1;
  }
  sockaddr_un a;
  socklen_t alen;
  make_addr(b->name, rank, &a, &alen);
  if (bind(b->listen_fd, reinterpret_cast<sockaddr*>(&a), alen) != 0 ||
      listen(b->listen_fd, 64) != 0) {
    set_last_error(std::string("broker: bind/listen: ") + strerror(errno));
    close(b->listen_fd);
    delete b;
    return -1;
  }
  std::string shm_name = "/" + b->name;
  const int64_t deadline = now_ms() + timeout_ms;
  if (rank == 0) {
    shm_unlink(shm_name.c_str());  // stale mailbox of a crashed job with the same name
    b->shm_fd = shm_open(shm_name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (b->shm_fd < 0 || ftruncate(b->shm_fd, sizeof(Mailbox)) != 0) {
      set_last_error(std::string("broker: shm_open/ftruncate: ") + strerror(errno));
      close(b->listen_fd);
      delete b;
      return -1;
    }
  } else {
    for (;;) {
      b->shm_fd = shm_open(shm_name.c_str(), O_RDWR, 0600);
      if (b->shm_fd >= 0) {
        struct stat st;
        if (fstat(b->shm_fd, &st) == 0 && size_t(st.st_size) >= sizeof(Mailbox)) break;
        close(b->shm_fd);
        b->shm_fd = -1;
      }
      if (now_ms() > deadline) {
        set_last_error("broker: timed out waiting for rank 0's mailbox");
        close(b->listen_fd);
        delete b;
        return -2;
      }
      usleep(1000);
    }
  }
  void* p = mmap(nullptr, sizeof(Mailbox), PROT_READ | PROT_WRITE, MAP_SHARED, b->shm_fd, 0);
  if (p == MAP_FAILED) {
    set_last_error(std::string("broker: mmap: ") + strerror(errno));
    close(b->listen_fd);
    close(b->shm_fd);
    delete b;
    return -1;
  }
  b->mb = static_cast<Mailbox*>(p);
  if (rank == 0) {
    // ftruncate zero-fills; publish readiness last.
    b->mb->ready.store(0x600dbeefu, std::memory_order_release);
  } else {
    while (b->mb->ready.load(std::memory_order_acquire) != 0x600dbeefu) {
      if (now_ms() > deadline) {
        set_last_error("broker: mailbox never became ready");
        munmap(b->mb, sizeof(Mailbox));
        close(b->listen_fd);
        close(b->shm_fd);
        delete b;
        return -2;
      }
      usleep(200);
    }
  }
  *out = b;
  return 0;
}

// Host barrier over the mailbox.  Returns -2 on time-out (a rank never came).
int cb_broker_barrier(void* broker, int timeout_ms) {
  Broker* b = static_cast<Broker*>(broker);
  const uint32_t round = b->barrier_round++;
  std::atomic<uint32_t>& ctr = b->mb->arrive[round & 1u];
  // Counter `round&1` is used every second round: it reaches world * (round/2 + 1).
  const uint32_t target = uint32_t(b->world) * (round / 2u + 1u);
  ctr.fetch_add(1, std::memory_order_acq_rel);
  const int64_t deadline = now_ms() + timeout_ms;
  uint32_t spins = 0;
  while (int32_t(ctr.load(std::memory_order_acquire) - target) < 0) {
    if ((++spins & 1023u) == 0) {
      if (now_ms() > deadline) {
        set_last_error("broker: barrier timed out (a rank did not arrive)");
        return -2;
      }
      usleep(50);
    }
  }
  return 0;
}

// All-gather of up to 256 bytes per rank through the mailbox.
int cb_broker_allgather(void* broker, const void* mine, int nbytes, void* all, int timeout_ms) {
  Broker* b = static_cast<Broker*>(broker);
  if (nbytes < 0 || nbytes > 256) {
    set_last_error("broker: allgather payload over 256 bytes");
    return -1;
  }
  int rc = cb_broker_barrier(b, timeout_ms);  // previous readers are done with the slots
  if (rc != 0) return rc;
  memcpy(b->mb->slots[b->rank], mine, size_t(nbytes));
  rc = cb_broker_barrier(b, timeout_ms);
  if (rc != 0) return rc;
  for (int r = 0; r < b->world; ++r)
    memcpy(static_cast<uint8_t*>(all) + size_t(r) * nbytes, b->mb->slots[r], size_t(nbytes));
  return 0;
}

// Every rank contributes one descriptor and receives everyone's
// (out_fds[rank] is a dup of its own).  Received descriptors belong to the caller.
int cb_broker_exchange_fds(void* broker, int my_fd, int* out_fds, int timeout_ms) {
  Broker* b = static_cast<Broker*>(broker);
  const uint32_t round = b->fd_round++;
  const int64_t deadline = now_ms() + timeout_ms;
  for (int r = 0; r < b->world; ++r) out_fds[r] = -1;
  out_fds[b->rank] = dup(my_fd);
  // 1. send to every peer (connect lands in the peer's backlog, so no peer has to be accepting).
  for (int p = 0; p < b->world; ++p) {
    if (p == b->rank) continue;
    sockaddr_un a;
    socklen_t alen;
    make_addr(b->name, p, &a, &alen);
    int s = -1;
    for (;;) {
      s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
      if (s >= 0 && connect(s, reinterpret_cast<sockaddr*>(&a), alen) == 0) break;
      if (s >= 0) close(s);
      s = -1;
      if (now_ms() > deadline) {
        set_last_error("broker: connect to rank " + std::to_string(p) + " timed out");
        return -2;
      }
      usleep(1000);
    }
    FdMsg m{round, b->rank};
    int rc = send_fd(s, m, my_fd);
    close(s);
    if (rc != 0) {
      set_last_error(std::string("broker: sendmsg: ") + strerror(errno));
      return -1;
    }
  }
  // 2. collect world-1 descriptors of this round.
  int have = 0;
  for (int p = 0; p < b->world; ++p) {
    if (p == b->rank) continue;
    auto it = b->pending.find({round, p});
    if (it != b->pending.end()) {
      out_fds[p] = it->second;
      b->pending.erase(it);
      ++have;
    }
  }
  while (have < b->world - 1) {
    pollfd pf{b->listen_fd, POLLIN, 0};
    int64_t left = deadline - now_ms();
    if (left <= 0 || poll(&pf, 1, int(left)) <= 0) {
      set_last_error("broker: timed out waiting for peers' descriptors");
      return -2;
    }
    int s = accept4(b->listen_fd, nullptr, nullptr, SOCK_CLOEXEC);
    if (s < 0) continue;
    FdMsg m;
    int fd = -1;
    pollfd ps{s, POLLIN, 0};
    int rc = -1;
    if (poll(&ps, 1, 2000) > 0) rc = recv_fd(s, &m, &fd);
    close(s);
    if (rc != 0) continue;
    if (m.src < 0 || m.src >= b->world) {
      close(fd);
      continue;
    }
    if (m.round == round && out_fds[m.src] < 0) {
      out_fds[m.src] = fd;
      ++have;
    } else {
      b->pending[{m.round, m.src}] = fd;
    }
  }
  return 0;
}

// Root's descriptor reaches every rank (out_fd on root is a dup of its own).
int cb_broker_broadcast_fd(void* broker, int root, int my_fd, int* out_fd, int timeout_ms) {
  Broker* b = static_cast<Broker*>(broker);
  // Non-root ranks contribute a harmless descriptor (their listening socket).
  int fds[CB_MAX_RANKS];
  int rc = cb_broker_exchange_fds(b, b->rank == root ? my_fd : b->listen_fd, fds, timeout_ms);
  if (rc != 0) return rc;
  for (int r = 0; r < b->world; ++r) {
    if (r == root) {
      *out_fd = fds[r];
    } else if (fds[r] >= 0) {
      close(fds[r]);
    }
  }
  return 0;
}

int cb_broker_destroy(void* broker) {
  Broker* b = static_cast<Broker*>(broker);
  if (b == nullptr) return 0;
  for (auto& kv : b->pending) close(kv.second);
  if (b->mb) munmap(b->mb, sizeof(Mailbox));
  if (b->shm_fd >= 0) close(b->shm_fd);
  if (b->listen_fd >= 0) close(b->listen_fd);
  if (b->rank == 0) shm_unlink(("/" + b->name).c_str());
  delete b;
  return 0;
}

}  // extern "C"
