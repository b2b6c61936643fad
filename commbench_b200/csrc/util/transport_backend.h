// Interface every transport backend implements; the C entry points of transport.h forward
// to one of these per open context.
#pragma once
#include <stdint.h>
#include <stdio.h>

#include <string>

#include "transport.h"

namespace cb {

class TransportBackend {
 public:
  virtual ~TransportBackend() = default;
  virtual int device_info_json(char* buf, int n) = 0;
  virtual int query_clock_ns(uint64_t* ns) = 0;
  virtual int reg_mr(void* addr, uint64_t len, int access, uint32_t* lkey, uint32_t* rkey) = 0;
  virtual int dereg_mr(uint32_t lkey) = 0;
  virtual int alloc_mw(uint32_t* id) = 0;
  virtual int mw_rkey(uint32_t id, uint32_t* rkey) = 0;
  virtual int dealloc_mw(uint32_t id) = 0;
  virtual int create_cq(int depth, uint32_t* cq) = 0;
  virtual int create_srq(int depth, uint32_t* srq) = 0;
  virtual int create_qp(int type, uint32_t send_cq, uint32_t recv_cq, uint32_t srq, int max_send_wr,
                        int max_recv_wr, int max_inline, CbTpAddr* local) = 0;
  virtual int query_max_inline(uint32_t qpn, int* v) = 0;
  virtual int connect(uint32_t qpn, const CbTpAddr* remote) = 0;
  virtual int destroy_qp(uint32_t qpn) = 0;
  virtual int post_recv(uint32_t qpn, uint64_t wr_id, const CbTpSge* sge, int n) = 0;
  virtual int post_srq_recv(uint32_t srq, uint64_t wr_id, const CbTpSge* sge, int n) = 0;
  virtual int post_send(uint32_t qpn, const CbTpSendWr* wr) = 0;
  virtual int poll_cq(uint32_t cq, CbTpCompletion* out, int max, int64_t timeout_us) = 0;
  virtual int get_async_event(int timeout_ms, int* event, uint32_t* object) = 0;
  virtual int ack_async_event() = 0;
};

// Defined in transport_verbs.cc: nullptr (and a reason in `why`) when libibverbs support was
// not compiled in or no device could be opened.
TransportBackend* open_verbs_backend(const char* device_name, std::string* why);
bool verbs_backend_compiled();

}  // namespace cb
