// Loopback backend of the transport API (see transport.h): all endpoints live in this
// process, work requests execute when they are posted.  Also holds the C entry points and
// dispatches to the verbs backend when a context was opened on it.
#include <cuda_runtime.h>
#include <string.h>
#include <time.h>

#include <chrono>
#include <condition_variable>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "transport.h"
#include "transport_backend.h"

namespace cb {
void set_last_error(const std::string& s);

namespace tplo {

struct Mr {
  uint8_t* base;
  uint64_t len;
  int access;
  bool device;     // GPU memory: touched only through cudaMemcpy
  bool window;     // a bound memory window (remote key only)
  uint32_t parent; // window: lkey of the region it is bound to
};

struct RecvWr {
  uint64_t wr_id;
  std::vector<CbTpSge> sge;
};

struct Cq {
  int depth;
  bool error = false;
  std::deque<CbTpCompletion> q;
};

struct Srq {
  int depth;
  std::deque<RecvWr> q;
};

struct PendingSend {   // RC send that found no receive posted yet
  uint32_t src_qpn;
  CbTpSendWr wr;
  std::vector<uint8_t> payload;
};

struct Qp {
  int type;
  uint32_t qpn;
  uint32_t send_cq, recv_cq, srq;
  int max_send_wr, max_recv_wr, max_inline;
  bool connected = false, error = false;
  CbTpAddr remote{};
  uint32_t qkey = 0;
  std::deque<RecvWr> rq;
  std::deque<PendingSend> waiting;   // sends from peers waiting for a receive (RC only)
};

uint64_t now_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return static_cast<uint64_t>(ts.tv_sec) * 1000000000ull + ts.tv_nsec;
}

bool is_device_ptr(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();  // no driver / not a CUDA pointer: plain host memory
    return false;
  }
  return a.type == cudaMemoryTypeDevice;
}

void copy_bytes(void* dst, bool dst_dev, const void* src, bool src_dev, size_t n) {
  if (n == 0) return;
  if (dst_dev || src_dev)
    cudaMemcpy(dst, src, n, cudaMemcpyDefault);
  else
    memcpy(dst, src, n);
}

class Loopback : public TransportBackend {
 public:
  explicit Loopback(std::string name) : name_(std::move(name)) {}

  int device_info_json(char* buf, int n) override {
    // Fixed field order: programs diff this output.
    int w = snprintf(
        buf, n,
        "{\"backend\": \"loopback\", \"device\": \"%s\", \"ports\": 1, \"port_state\": \"ACTIVE\", "
        "\"link_layer\": \"loopback\", \"mtu\": %d, \"max_qp\": 65536, \"max_cq\": 65536, "
        "\"max_mr\": 1048576, \"max_sge\": %d, \"max_inline\": 1024, \"max_srq\": 4096, "
        "\"atomic_cap\": \"ATOMIC_GLOB\", \"gid\": \"00000000000000000000ffff7f000001\", "
        "\"data_in_order\": {\"RC\": {\"SEND\": true, \"WRITE\": true, \"WRITE_IMM\": true}, "
        "\"UC\": {\"SEND\": true, \"WRITE\": true, \"WRITE_IMM\": true}, "
        "\"UD\": {\"SEND\": true, \"WRITE\": false, \"WRITE_IMM\": false}}}",
        name_.c_str(), CB_TP_UD_MTU, CB_TP_MAX_SGE);
    return (w > 0 && w < n) ? w : -1;
  }

  int query_clock_ns(uint64_t* ns) override {
    *ns = now_ns();
    return 0;
  }

  // ---------------------------------------------------------------------------- memory
  int reg_mr(void* addr, uint64_t len, int access, uint32_t* lkey, uint32_t* rkey) override {
    std::lock_guard<std::mutex> g(mu_);
    if (addr == nullptr || len == 0) return fail("reg_mr: empty region");
    if ((access & (CB_TP_REMOTE_WRITE | CB_TP_REMOTE_ATOMIC)) && !(access & CB_TP_LOCAL_WRITE))
      return fail("reg_mr: remote write / atomic access requires local write access");
    const uint32_t key = next_key_++;
    mrs_[key] = Mr{static_cast<uint8_t*>(addr), len, access, is_device_ptr(addr), false, 0};
    *lkey = key;
    *rkey = key;   // one key space; windows get keys of their own
    return 0;
  }
  int dereg_mr(uint32_t lkey) override {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& kv : mrs_)
      if (kv.second.window && kv.second.parent == lkey)
        return fail("dereg_mr: a memory window is still bound to this region");
    return mrs_.erase(lkey) ? 0 : fail("dereg_mr: unknown key");
  }
  int alloc_mw(uint32_t* id) override {
    std::lock_guard<std::mutex> g(mu_);
    *id = next_mw_++;
    mws_[*id] = 0;
    return 0;
  }
  int mw_rkey(uint32_t id, uint32_t* rkey) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = mws_.find(id);
    if (it == mws_.end() || it->second == 0) return fail("mw_rkey: window is not bound");
    *rkey = it->second;
    return 0;
  }
  int dealloc_mw(uint32_t id) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = mws_.find(id);
    if (it == mws_.end()) return fail("dealloc_mw: unknown window");
    if (it->second) mrs_.erase(it->second);
    mws_.erase(it);
    return 0;
  }

  // ---------------------------------------------------------------------------- queues
  int create_cq(int depth, uint32_t* cq) override {
    std::lock_guard<std::mutex> g(mu_);
    if (depth < 1) return fail("create_cq: depth must be positive");
    *cq = next_obj_++;
    cqs_[*cq].depth = depth;
    cq_owner_[*cq] = this;
    return 0;
  }
  int create_srq(int depth, uint32_t* srq) override {
    std::lock_guard<std::mutex> g(mu_);
    if (depth < 1) return fail("create_srq: depth must be positive");
    *srq = next_obj_++;
    srqs_[*srq].depth = depth;
    return 0;
  }
  int create_qp(int type, uint32_t send_cq, uint32_t recv_cq, uint32_t srq, int max_send_wr,
                int max_recv_wr, int max_inline, CbTpAddr* local) override {
    std::lock_guard<std::mutex> g(mu_);
    if (type < CB_TP_RC || type > CB_TP_UD) return fail("create_qp: bad type");
    if (!cqs_.count(send_cq) || !cqs_.count(recv_cq)) return fail("create_qp: unknown completion queue");
    if (srq != 0 && !srqs_.count(srq)) return fail("create_qp: unknown shared receive queue");
    if (max_inline > 1024) return fail("create_qp: max_inline above the device limit (1024)");
    Qp q;
    q.type = type;
    q.qpn = next_qpn_++;
    q.send_cq = send_cq;
    q.recv_cq = recv_cq;
    q.srq = srq;
    q.max_send_wr = max_send_wr;
    q.max_recv_wr = max_recv_wr;
    q.max_inline = max_inline < 0 ? 0 : max_inline;
    q.qkey = 0x11111111u;
    memset(local, 0, sizeof(*local));
    local->qpn = q.qpn;
    local->psn = (q.qpn * 2654435761u) & 0xffffffu;
    local->qkey = q.qkey;
    local->lid = 1;
    local->gid[10] = 0xff;
    local->gid[11] = 0xff;
    local->gid[12] = 127;
    local->gid[15] = 1;
    qps_[q.qpn] = std::move(q);
    return 0;
  }
  int query_max_inline(uint32_t qpn, int* v) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = qps_.find(qpn);
    if (it == qps_.end()) return fail("query_max_inline: unknown queue pair");
    *v = it->second.max_inline;
    return 0;
  }
  int connect(uint32_t qpn, const CbTpAddr* remote) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = qps_.find(qpn);
    if (it == qps_.end()) return fail("connect: unknown queue pair");
    if (it->second.type != CB_TP_UD) {
      if (remote == nullptr) return fail("connect: a connected queue pair needs the peer's address");
      it->second.remote = *remote;
    }
    it->second.connected = true;
    return 0;
  }
  int destroy_qp(uint32_t qpn) override {
    std::lock_guard<std::mutex> g(mu_);
    if (unacked_ > 0 && last_event_obj_ == qpn)
      return fail("destroy_qp: an asynchronous event naming this queue pair is not acknowledged");
    return qps_.erase(qpn) ? 0 : fail("destroy_qp: unknown queue pair");
  }

  int post_recv(uint32_t qpn, uint64_t wr_id, const CbTpSge* sge, int n) override;
  int post_srq_recv(uint32_t srq, uint64_t wr_id, const CbTpSge* sge, int n) override;
  int post_send(uint32_t qpn, const CbTpSendWr* wr) override;
  int poll_cq(uint32_t cq, CbTpCompletion* out, int max, int64_t timeout_us) override;
  int get_async_event(int timeout_ms, int* event, uint32_t* object) override;
  int ack_async_event() override;

 private:
  int fail(const std::string& why) {
    set_last_error("transport(loopback): " + why);
    return -1;
  }
  // Looks up a key and checks [addr, addr+len) and the access bits.
  Mr* check(uint32_t key, uint64_t addr, uint64_t len, int need) {
    auto it = mrs_.find(key);
    if (it == mrs_.end()) return nullptr;
    Mr& m = it->second;
    const uint64_t b = reinterpret_cast<uint64_t>(m.base);
    if (addr < b || addr + len > b + m.len || addr + len < addr) return nullptr;
    if ((m.access & need) != need) return nullptr;
    return &m;
  }
  void complete(uint32_t cq_id, const CbTpCompletion& c);
  bool gather(const Qp& q, const CbTpSendWr& wr, std::vector<uint8_t>* out, int* status);
  int scatter(const RecvWr& r, const uint8_t* data, size_t n, size_t prefix);
  bool take_recv(Qp& dst, RecvWr* out);
  void deliver(Qp& dst, uint32_t src_qpn, const CbTpSendWr& wr, const std::vector<uint8_t>& payload,
               const RecvWr& r);
  void raise(int event, uint32_t object);

  std::string name_;
  // One fabric per process: every loopback context sees every queue pair and key, so two
  // contexts ("two adapters") can talk to each other.  One lock serialises all operations.
  static inline std::mutex mu_;
  static inline std::condition_variable cv_;
  static inline std::map<uint32_t, Mr> mrs_;
  static inline std::map<uint32_t, uint32_t> mws_;   // window id -> bound remote key (0 = unbound)
  static inline std::map<uint32_t, Cq> cqs_;
  static inline std::map<uint32_t, Srq> srqs_;
  static inline std::map<uint32_t, Qp> qps_;
  static inline uint32_t next_key_ = 0x1000, next_mw_ = 1, next_obj_ = 1, next_qpn_ = 0x100;
  // Asynchronous events are per context (per "adapter").
  std::deque<std::pair<int, uint32_t>> events_;
  int unacked_ = 0;
  uint32_t last_event_obj_ = 0;
  std::map<uint32_t, bool> my_cqs_;   // completion queues created through this context
  static inline std::map<uint32_t, Loopback*> cq_owner_;
};

#include "transport_loopback_ops.inc"

}  // namespace tplo
using tplo::Loopback;
}  // namespace cb

#include "transport_capi.inc"
