// libibverbs backend of the transport API.  Compiled only when the verbs header exists on
// the build machine; otherwise opening it reports that it was not built.  The structure follows
// the usual verbs life cycle the reference's endpoints implement by hand
// (datasets/example002_rdma_loopback/empty_rdma_loopback.cpp:142-390: device, protection domain,
// completion queue, memory region, queue pair INIT -> RTR -> RTS, post, poll).
#include <string>

#include "transport_backend.h"

#if defined(__has_include)
#if __has_include(<infiniband/verbs.h>)
#define CB_HAVE_VERBS 1
#endif
#endif

#ifndef CB_HAVE_VERBS

namespace cb {
bool verbs_backend_compiled() { return false; }
TransportBackend* open_verbs_backend(const char*, std::string* why) {
  *why = "this build has no libibverbs support (infiniband/verbs.h was not found at build time)";
  return nullptr;
}
}  // namespace cb

#else  // ------------------------------------------------------------------ real backend

#include <infiniband/verbs.h>
#include <poll.h>
#include <string.h>

#include <map>
#include <mutex>
#include <vector>

namespace cb {
void set_last_error(const std::string& s);
bool verbs_backend_compiled() { return true; }

namespace {

class Verbs : public TransportBackend {
 public:
  ~Verbs() override {
    for (ibv_ah* ah : ahs_) ibv_destroy_ah(ah);
    for (auto& kv : qps_) ibv_destroy_qp(kv.second);
    for (auto& kv : srqs_) ibv_destroy_srq(kv.second);
    for (auto& kv : cqs_) ibv_destroy_cq(kv.second);
    for (auto& kv : mws_) ibv_dealloc_mw(kv.second);
    for (auto& kv : mrs_) ibv_dereg_mr(kv.second);
    if (pd_) ibv_dealloc_pd(pd_);
    if (ctx_) ibv_close_device(ctx_);
  }

  bool open(const char* name, std::string* why) {
    int n = 0;
    ibv_device** list = ibv_get_device_list(&n);
    if (list == nullptr || n == 0) {
      *why = "no RDMA device";
      return false;
    }
    ibv_device* dev = list[0];
    for (int i = 0; i < n; ++i)
      if (name && *name && strcmp(ibv_get_device_name(list[i]), name) == 0) dev = list[i];
    ctx_ = ibv_open_device(dev);
    name_ = ibv_get_device_name(dev);
    ibv_free_device_list(list);
    if (!ctx_) {
      *why = "ibv_open_device failed";
      return false;
    }
    pd_ = ibv_alloc_pd(ctx_);
    if (!pd_ || ibv_query_port(ctx_, 1, &port_) != 0 || ibv_query_device(ctx_, &attr_) != 0) {
      *why = "protection domain / port query failed";
      return false;
    }
    ibv_query_gid(ctx_, 1, 0, &gid_);
    return true;
  }

  int device_info_json(char* buf, int n) override {
    char gid[33];
    for (int i = 0; i < 16; ++i) snprintf(gid + 2 * i, 3, "%02x", gid_.raw[i]);
    const char* atomic = attr_.atomic_cap == IBV_ATOMIC_GLOB   ? "ATOMIC_GLOB"
                         : attr_.atomic_cap == IBV_ATOMIC_HCA ? "ATOMIC_HCA"
                                                              : "ATOMIC_NONE";
    int w = snprintf(buf, n,
                     "{\"backend\": \"verbs\", \"device\": \"%s\", \"ports\": %d, \"port_state\": \"%s\", "
                     "\"link_layer\": \"%s\", \"mtu\": %d, \"max_qp\": %d, \"max_cq\": %d, \"max_mr\": %d, "
                     "\"max_sge\": %d, \"max_srq\": %d, \"atomic_cap\": \"%s\", \"gid\": \"%s\"}",
                     name_.c_str(), attr_.phys_port_cnt, ibv_port_state_str(port_.state),
                     port_.link_layer == IBV_LINK_LAYER_ETHERNET ? "Ethernet" : "InfiniBand",
                     128 << port_.active_mtu, attr_.max_qp, attr_.max_cq, attr_.max_mr, attr_.max_sge,
                     attr_.max_srq, atomic, gid);
    return (w > 0 && w < n) ? w : -1;
  }

  int query_clock_ns(uint64_t* ns) override {
    ibv_values_ex v{};
    v.comp_mask = IBV_VALUES_MASK_RAW_CLOCK;
    if (ibv_query_rt_values_ex(ctx_, &v) != 0) return fail("ibv_query_rt_values_ex");
    *ns = static_cast<uint64_t>(v.raw_clock.tv_sec) * 1000000000ull + v.raw_clock.tv_nsec;
    return 0;
  }

  int reg_mr(void* addr, uint64_t len, int access, uint32_t* lkey, uint32_t* rkey) override {
    int a = 0;
    if (access & CB_TP_LOCAL_WRITE) a |= IBV_ACCESS_LOCAL_WRITE;
    if (access & CB_TP_REMOTE_WRITE) a |= IBV_ACCESS_REMOTE_WRITE;
    if (access & CB_TP_REMOTE_READ) a |= IBV_ACCESS_REMOTE_READ;
    if (access & CB_TP_REMOTE_ATOMIC) a |= IBV_ACCESS_REMOTE_ATOMIC;
    if (access & CB_TP_MW_BIND) a |= IBV_ACCESS_MW_BIND;
    ibv_mr* mr = ibv_reg_mr(pd_, addr, len, a);   // GPU memory works when peer-memory support is loaded
    if (!mr) return fail("ibv_reg_mr");
    std::lock_guard<std::mutex> g(mu_);
    mrs_[mr->lkey] = mr;
    *lkey = mr->lkey;
    *rkey = mr->rkey;
    return 0;
  }
  int dereg_mr(uint32_t lkey) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = mrs_.find(lkey);
    if (it == mrs_.end()) return fail("dereg_mr: unknown key");
    ibv_dereg_mr(it->second);
    mrs_.erase(it);
    return 0;
  }
  int alloc_mw(uint32_t* id) override {
    ibv_mw* mw = ibv_alloc_mw(pd_, IBV_MW_TYPE_2);
    if (!mw) return fail("ibv_alloc_mw");
    std::lock_guard<std::mutex> g(mu_);
    *id = next_id_++;
    mws_[*id] = mw;
    return 0;
  }
  int mw_rkey(uint32_t id, uint32_t* rkey) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = mws_.find(id);
    if (it == mws_.end()) return fail("mw_rkey: unknown window");
    *rkey = it->second->rkey;
    return 0;
  }
  int dealloc_mw(uint32_t id) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = mws_.find(id);
    if (it == mws_.end()) return fail("dealloc_mw: unknown window");
    ibv_dealloc_mw(it->second);
    mws_.erase(it);
    return 0;
  }

  int create_cq(int depth, uint32_t* cq) override {
    ibv_cq* c = ibv_create_cq(ctx_, depth, nullptr, nullptr, 0);
    if (!c) return fail("ibv_create_cq");
    std::lock_guard<std::mutex> g(mu_);
    *cq = next_id_++;
    cqs_[*cq] = c;
    return 0;
  }
  int create_srq(int depth, uint32_t* srq) override {
    ibv_srq_init_attr a{};
    a.attr.max_wr = depth;
    a.attr.max_sge = CB_TP_MAX_SGE;
    ibv_srq* s = ibv_create_srq(pd_, &a);
    if (!s) return fail("ibv_create_srq");
    std::lock_guard<std::mutex> g(mu_);
    *srq = next_id_++;
    srqs_[*srq] = s;
    return 0;
  }
  int create_qp(int type, uint32_t send_cq, uint32_t recv_cq, uint32_t srq, int max_send_wr,
                int max_recv_wr, int max_inline, CbTpAddr* local) override {
    std::lock_guard<std::mutex> g(mu_);
    ibv_qp_init_attr a{};
    a.qp_type = type == CB_TP_RC ? IBV_QPT_RC : type == CB_TP_UC ? IBV_QPT_UC : IBV_QPT_UD;
    a.send_cq = cqs_.at(send_cq);
    a.recv_cq = cqs_.at(recv_cq);
    a.srq = srq ? srqs_.at(srq) : nullptr;
    a.cap.max_send_wr = max_send_wr;
    a.cap.max_recv_wr = max_recv_wr;
    a.cap.max_send_sge = CB_TP_MAX_SGE;
    a.cap.max_recv_sge = CB_TP_MAX_SGE;
    a.cap.max_inline_data = max_inline;
    ibv_qp* qp = ibv_create_qp(pd_, &a);
    if (!qp) return fail("ibv_create_qp");
    ibv_qp_attr m{};
    m.qp_state = IBV_QPS_INIT;
    m.port_num = 1;
    int mask = IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT;
    if (type == CB_TP_UD) {
      m.qkey = 0x11111111u;
      mask |= IBV_QP_QKEY;
    } else {
      m.qp_access_flags = IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ | IBV_ACCESS_REMOTE_ATOMIC;
      mask |= IBV_QP_ACCESS_FLAGS;
    }
    if (ibv_modify_qp(qp, &m, mask) != 0) {
      ibv_destroy_qp(qp);
      return fail("ibv_modify_qp(INIT)");
    }
    qps_[qp->qp_num] = qp;
    types_[qp->qp_num] = type;
    inline_[qp->qp_num] = a.cap.max_inline_data;
    memset(local, 0, sizeof(*local));
    local->qpn = qp->qp_num;
    local->psn = (qp->qp_num * 2654435761u) & 0xffffffu;
    local->qkey = 0x11111111u;
    local->lid = port_.lid;
    memcpy(local->gid, gid_.raw, 16);
    return 0;
  }
  int query_max_inline(uint32_t qpn, int* v) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = inline_.find(qpn);
    if (it == inline_.end()) return fail("query_max_inline: unknown queue pair");
    *v = static_cast<int>(it->second);
    return 0;
  }
  int connect(uint32_t qpn, const CbTpAddr* r) override {
    std::lock_guard<std::mutex> g(mu_);
    ibv_qp* qp = qps_.at(qpn);
    const int type = types_.at(qpn);
    ibv_qp_attr a{};
    a.qp_state = IBV_QPS_RTR;
    int mask = IBV_QP_STATE;
    if (type != CB_TP_UD) {
      a.path_mtu = port_.active_mtu;
      a.dest_qp_num = r->qpn;
      a.rq_psn = r->psn;
      a.ah_attr.dlid = static_cast<uint16_t>(r->lid);
      a.ah_attr.port_num = 1;
      a.ah_attr.is_global = 1;
      memcpy(a.ah_attr.grh.dgid.raw, r->gid, 16);
      a.ah_attr.grh.hop_limit = 1;
      mask |= IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN;
      if (type == CB_TP_RC) {
        a.max_dest_rd_atomic = 1;
        a.min_rnr_timer = 12;
        mask |= IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER;
      }
    }
    if (ibv_modify_qp(qp, &a, mask) != 0) return fail("ibv_modify_qp(RTR)");
    ibv_qp_attr s{};
    s.qp_state = IBV_QPS_RTS;
    s.sq_psn = (qpn * 2654435761u) & 0xffffffu;
    mask = IBV_QP_STATE | IBV_QP_SQ_PSN;
    if (type == CB_TP_RC) {
      s.timeout = 14;
      s.retry_cnt = 7;
      s.rnr_retry = 7;
      s.max_rd_atomic = 1;
      mask |= IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_MAX_QP_RD_ATOMIC;
    }
    if (ibv_modify_qp(qp, &s, mask) != 0) return fail("ibv_modify_qp(RTS)");
    return 0;
  }
  int destroy_qp(uint32_t qpn) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = qps_.find(qpn);
    if (it == qps_.end()) return fail("destroy_qp: unknown queue pair");
    ibv_destroy_qp(it->second);
    qps_.erase(it);
    return 0;
  }

  static void to_sge(const CbTpSge* in, int n, ibv_sge* out) {
    for (int i = 0; i < n; ++i) {
      out[i].addr = in[i].addr;
      out[i].length = in[i].length;
      out[i].lkey = in[i].lkey;
    }
  }
  int post_recv(uint32_t qpn, uint64_t wr_id, const CbTpSge* sge, int n) override {
    ibv_sge s[CB_TP_MAX_SGE];
    to_sge(sge, n, s);
    ibv_recv_wr wr{}, *bad = nullptr;
    wr.wr_id = wr_id;
    wr.sg_list = s;
    wr.num_sge = n;
    return ibv_post_recv(qps_.at(qpn), &wr, &bad) == 0 ? 0 : fail("ibv_post_recv");
  }
  int post_srq_recv(uint32_t srq, uint64_t wr_id, const CbTpSge* sge, int n) override {
    ibv_sge s[CB_TP_MAX_SGE];
    to_sge(sge, n, s);
    ibv_recv_wr wr{}, *bad = nullptr;
    wr.wr_id = wr_id;
    wr.sg_list = s;
    wr.num_sge = n;
    return ibv_post_srq_recv(srqs_.at(srq), &wr, &bad) == 0 ? 0 : fail("ibv_post_srq_recv");
  }
  int post_send(uint32_t qpn, const CbTpSendWr* w) override {
    ibv_qp* qp = qps_.at(qpn);
    if (w->opcode == CB_TP_BIND_MW) {
      ibv_mw_bind b{};
      b.wr_id = w->wr_id;
      b.send_flags = (w->flags & CB_TP_SIGNALED) ? IBV_SEND_SIGNALED : 0;
      b.bind_info.mr = mrs_.at(w->bind_lkey);
      b.bind_info.addr = w->bind_addr;
      b.bind_info.length = w->bind_length;
      b.bind_info.mw_access_flags =
          ((w->bind_access & CB_TP_REMOTE_WRITE) ? IBV_ACCESS_REMOTE_WRITE : 0) |
          ((w->bind_access & CB_TP_REMOTE_READ) ? IBV_ACCESS_REMOTE_READ : 0);
      return ibv_bind_mw(qp, mws_.at(w->mw_id), &b) == 0 ? 0 : fail("ibv_bind_mw");
    }
    ibv_sge s[CB_TP_MAX_SGE];
    to_sge(w->sge, w->num_sge, s);
    ibv_send_wr wr{}, *bad = nullptr;
    wr.wr_id = w->wr_id;
    wr.sg_list = s;
    wr.num_sge = w->num_sge;
    wr.send_flags = ((w->flags & CB_TP_SIGNALED) ? IBV_SEND_SIGNALED : 0) |
                    ((w->flags & CB_TP_INLINE) ? IBV_SEND_INLINE : 0);
    wr.imm_data = w->imm;
    ibv_ah* ah = nullptr;
    switch (w->opcode) {
      case CB_TP_SEND: wr.opcode = IBV_WR_SEND; break;
      case CB_TP_SEND_IMM: wr.opcode = IBV_WR_SEND_WITH_IMM; break;
      case CB_TP_WRITE: wr.opcode = IBV_WR_RDMA_WRITE; break;
      case CB_TP_WRITE_IMM: wr.opcode = IBV_WR_RDMA_WRITE_WITH_IMM; break;
      case CB_TP_READ: wr.opcode = IBV_WR_RDMA_READ; break;
      case CB_TP_ATOMIC_CAS: wr.opcode = IBV_WR_ATOMIC_CMP_AND_SWP; break;
      case CB_TP_ATOMIC_FADD: wr.opcode = IBV_WR_ATOMIC_FETCH_AND_ADD; break;
      case CB_TP_LOCAL_INV:
        wr.opcode = IBV_WR_LOCAL_INV;
        wr.invalidate_rkey = w->mw_id;
        break;
      default: return fail("post_send: bad opcode");
    }
    if (w->opcode == CB_TP_ATOMIC_CAS || w->opcode == CB_TP_ATOMIC_FADD) {
      wr.wr.atomic.remote_addr = w->remote_addr;
      wr.wr.atomic.rkey = w->rkey;
      wr.wr.atomic.compare_add = w->compare_add;
      wr.wr.atomic.swap = w->swap;
    } else if (types_.at(qpn) == CB_TP_UD) {
      ibv_ah_attr a{};
      a.dlid = static_cast<uint16_t>(w->ud_dest.lid);
      a.port_num = 1;
      a.is_global = 1;
      memcpy(a.grh.dgid.raw, w->ud_dest.gid, 16);
      a.grh.hop_limit = 1;
      ah = ibv_create_ah(pd_, &a);
      if (!ah) return fail("ibv_create_ah");
      wr.wr.ud.ah = ah;
      wr.wr.ud.remote_qpn = w->ud_dest.qpn;
      wr.wr.ud.remote_qkey = w->ud_dest.qkey;
    } else {
      wr.wr.rdma.remote_addr = w->remote_addr;
      wr.wr.rdma.rkey = w->rkey;
    }
    const int rc = ibv_post_send(qp, &wr, &bad);
    if (ah) ahs_.push_back(ah);   // must outlive the send; freed with the context
    return rc == 0 ? 0 : fail("ibv_post_send");
  }
  int poll_cq(uint32_t cq, CbTpCompletion* out, int max, int64_t timeout_us) override {
    ibv_cq* c = cqs_.at(cq);
    std::vector<ibv_wc> wc(max);
    timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (;;) {
      const int n = ibv_poll_cq(c, max, wc.data());
      if (n < 0) return fail("ibv_poll_cq");
      if (n > 0) {
        for (int i = 0; i < n; ++i) {
          out[i] = CbTpCompletion{};
          out[i].wr_id = wc[i].wr_id;
          out[i].status = wc[i].status == IBV_WC_SUCCESS ? CB_TP_OK : map_status(wc[i].status);
          out[i].opcode = (wc[i].opcode & IBV_WC_RECV)
                              ? ((wc[i].wc_flags & IBV_WC_WITH_IMM) ? CB_TP_RECV_IMM : CB_TP_RECV)
                              : CB_TP_SEND;
          out[i].byte_len = wc[i].byte_len;
          out[i].imm = wc[i].imm_data;
          out[i].src_qpn = wc[i].src_qp;
          out[i].qpn = wc[i].qp_num;
        }
        return n;
      }
      timespec t1;
      clock_gettime(CLOCK_MONOTONIC, &t1);
      const int64_t us = (t1.tv_sec - t0.tv_sec) * 1000000ll + (t1.tv_nsec - t0.tv_nsec) / 1000;
      if (us >= timeout_us) return 0;
    }
  }
  int get_async_event(int timeout_ms, int* event, uint32_t* object) override {
    pollfd p{ctx_->async_fd, POLLIN, 0};
    if (poll(&p, 1, timeout_ms) <= 0) {
      *event = CB_TP_EVENT_NONE;
      *object = 0;
      return 0;
    }
    if (ibv_get_async_event(ctx_, &pending_) != 0) return fail("ibv_get_async_event");
    have_pending_ = true;
    *event = pending_.event_type == IBV_EVENT_CQ_ERR ? CB_TP_EVENT_CQ_ERR : CB_TP_EVENT_QP_FATAL;
    *object = 0;
    return 1;
  }
  int ack_async_event() override {
    if (!have_pending_) return fail("ack_async_event: nothing to acknowledge");
    ibv_ack_async_event(&pending_);
    have_pending_ = false;
    return 0;
  }

 private:
  static int map_status(int s) {
    switch (s) {
      case IBV_WC_LOC_LEN_ERR: return CB_TP_LOC_LEN_ERR;
      case IBV_WC_LOC_PROT_ERR: return CB_TP_LOC_PROT_ERR;
      case IBV_WC_REM_ACCESS_ERR: return CB_TP_REM_ACCESS_ERR;
      case IBV_WC_REM_INV_REQ_ERR: return CB_TP_REM_INV_REQ_ERR;
      case IBV_WC_RNR_RETRY_EXC_ERR: return CB_TP_RNR_RETRY_EXC;
      default: return CB_TP_WR_FLUSH_ERR;
    }
  }
  int fail(const std::string& what) {
    set_last_error("transport(verbs): " + what + " failed");
    return -1;
  }
  ibv_context* ctx_ = nullptr;
  ibv_pd* pd_ = nullptr;
  ibv_port_attr port_{};
  ibv_device_attr attr_{};
  ibv_gid gid_{};
  std::string name_;
  std::mutex mu_;
  std::map<uint32_t, ibv_mr*> mrs_;
  std::map<uint32_t, ibv_mw*> mws_;
  std::map<uint32_t, ibv_cq*> cqs_;
  std::map<uint32_t, ibv_srq*> srqs_;
  std::map<uint32_t, ibv_qp*> qps_;
  std::map<uint32_t, int> types_;
  std::map<uint32_t, uint32_t> inline_;
  std::vector<ibv_ah*> ahs_;
  ibv_async_event pending_{};
  bool have_pending_ = false;
  uint32_t next_id_ = 1;
};

}  // namespace

TransportBackend* open_verbs_backend(const char* device_name, std::string* why) {
  Verbs* v = new Verbs();
  if (!v->open(device_name, why)) {
    delete v;
    return nullptr;
  }
  return v;
}

}  // namespace cb

#endif
