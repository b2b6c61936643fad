// Host-side message transport with verbs-like semantics: endpoints (queue pairs) of type
// RC / UC / UD, registered memory regions with local and remote keys, completion queues,
// shared receive queues, memory windows, one-sided WRITE / READ / atomics, two-sided
// SEND / RECV with immediate data, inline and scatter-gather sends, asynchronous error
// events and a device clock.
//
// Two backends implement the same C ABI:
//   * loopback - every endpoint lives in this process; operations execute at post time on
//                the registered buffers (host memory, or device memory through cudaMemcpy).
//                It keeps the verbs rules that programs depend on: a SEND or WRITE_WITH_IMM
//                consumes a posted receive, UC has no READ / atomics, UD carries at most
//                one MTU and prefixes 40 bytes, unsignalled sends complete silently, remote
//                keys and bounds are checked, a full completion queue raises an
//                asynchronous CQ error.
//   * verbs    - libibverbs, compiled only when <infiniband/verbs.h> is present.
//
// The reference's RDMA family (datasets/example002_rdma_loopback/empty_rdma_loopback.cpp:
// 142-390 `RdmaEndpoint`; example006 RC write with metadata exchange; example007 UC send/recv;
// example008 shared receive queue; example011/013 write-with-immediate; example014 inline;
// example015 memory pool; example016 UD; example019 scatter-gather; example024/025 atomics;
// example026 asynchronous events; example027 memory windows; example028 device clock;
// example029 in-order query; example004 device info) is written against raw libibverbs; this
// header is the one API all of those patterns are expressed in here.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum CbTpBackend { CB_TP_LOOPBACK = 0, CB_TP_VERBS = 1 };
enum CbTpQpType { CB_TP_RC = 0, CB_TP_UC = 1, CB_TP_UD = 2 };
enum CbTpOpcode {
  CB_TP_SEND = 0,
  CB_TP_SEND_IMM = 1,
  CB_TP_WRITE = 2,
  CB_TP_WRITE_IMM = 3,
  CB_TP_READ = 4,
  CB_TP_ATOMIC_CAS = 5,
  CB_TP_ATOMIC_FADD = 6,
  CB_TP_BIND_MW = 7,
  CB_TP_LOCAL_INV = 8,
  CB_TP_RECV = 64,          // completion opcodes of the receive side
  CB_TP_RECV_IMM = 65,
};
enum CbTpAccess {
  CB_TP_LOCAL_WRITE = 1,
  CB_TP_REMOTE_WRITE = 2,
  CB_TP_REMOTE_READ = 4,
  CB_TP_REMOTE_ATOMIC = 8,
  CB_TP_MW_BIND = 16,
};
enum CbTpSendFlags { CB_TP_SIGNALED = 1, CB_TP_INLINE = 2 };
enum CbTpStatus {
  CB_TP_OK = 0,
  CB_TP_LOC_LEN_ERR = 1,      // receive buffer too small / bad local length
  CB_TP_LOC_PROT_ERR = 2,     // bad local key or range
  CB_TP_REM_ACCESS_ERR = 3,   // bad remote key, range or permission
  CB_TP_REM_INV_REQ_ERR = 4,  // operation not valid on this queue-pair type / state
  CB_TP_RNR_RETRY_EXC = 5,    // no receive posted (RC, retries exhausted)
  CB_TP_WR_FLUSH_ERR = 6,     // queue pair in error state
};
enum CbTpEvent { CB_TP_EVENT_NONE = 0, CB_TP_EVENT_CQ_ERR = 1, CB_TP_EVENT_QP_FATAL = 2 };

#define CB_TP_MAX_SGE 16
#define CB_TP_UD_HEADER 40   // bytes a UD receive buffer loses to the routing header
#define CB_TP_UD_MTU 4096

typedef struct {
  uint64_t addr;
  uint32_t length;
  uint32_t lkey;
} CbTpSge;

// Everything a peer needs to reach a queue pair (what programs exchange over TCP).
typedef struct {
  uint32_t qpn;
  uint32_t psn;
  uint32_t qkey;      // UD only
  uint32_t lid;
  uint8_t gid[16];
} CbTpAddr;

typedef struct {
  uint64_t wr_id;
  int opcode;           // CbTpOpcode
  int flags;            // CbTpSendFlags
  int num_sge;
  CbTpSge sge[CB_TP_MAX_SGE];
  uint32_t imm;
  uint64_t remote_addr;
  uint32_t rkey;
  uint64_t compare_add; // CAS: compare value; FADD: addend
  uint64_t swap;        // CAS: swap value
  CbTpAddr ud_dest;     // UD: destination of this datagram
  // BIND_MW / LOCAL_INV
  uint32_t mw_id;       // window to bind or rkey to invalidate
  uint32_t bind_lkey;   // region the window is bound to
  uint64_t bind_addr;
  uint64_t bind_length;
  int bind_access;
} CbTpSendWr;

typedef struct {
  uint64_t wr_id;
  int status;           // CbTpStatus
  int opcode;           // CbTpOpcode (send side: the posted opcode; receive side: RECV / RECV_IMM)
  uint32_t byte_len;
  uint32_t imm;
  uint32_t src_qpn;
  uint32_t qpn;
} CbTpCompletion;

// --- context / device ------------------------------------------------------------------
// Returns a context handle (> 0) or 0 (see cb_last_error()).
uint64_t cb_tp_open(int backend, const char* device_name);
void cb_tp_close(uint64_t ctx);
// Deterministic JSON description of the device (ports, MTU, limits, atomic capability,
// per queue-pair-type "data written in order" flags).  Returns bytes written or -1.
int cb_tp_device_info_json(uint64_t ctx, char* buf, int buf_len);
int cb_tp_backend_available(int backend);
// Device clock in nanoseconds (monotonic) - the analogue of a NIC's free-running counter.
int cb_tp_query_clock_ns(uint64_t ctx, uint64_t* ns);

// --- memory ----------------------------------------------------------------------------
// Registers [addr, addr+len).  `is_device` = memory on a GPU (copied with cudaMemcpy).
int cb_tp_reg_mr(uint64_t ctx, void* addr, uint64_t len, int access, uint32_t* lkey, uint32_t* rkey);
int cb_tp_dereg_mr(uint64_t ctx, uint32_t lkey);
// Memory windows: allocate, then bind through a BIND_MW work request; the new remote key is
// returned here after the bind completed.
int cb_tp_alloc_mw(uint64_t ctx, uint32_t* mw_id);
int cb_tp_mw_rkey(uint64_t ctx, uint32_t mw_id, uint32_t* rkey);
int cb_tp_dealloc_mw(uint64_t ctx, uint32_t mw_id);

// --- queues ----------------------------------------------------------------------------
int cb_tp_create_cq(uint64_t ctx, int depth, uint32_t* cq);
int cb_tp_create_srq(uint64_t ctx, int depth, uint32_t* srq);
// `srq` = 0 for a private receive queue.
int cb_tp_create_qp(uint64_t ctx, int type, uint32_t send_cq, uint32_t recv_cq, uint32_t srq,
                    int max_send_wr, int max_recv_wr, int max_inline, CbTpAddr* local);
int cb_tp_query_max_inline(uint64_t ctx, uint32_t qpn, int* max_inline);
// RC / UC: connect to the peer (INIT -> RTR -> RTS).  UD: only moves the QP to RTS.
int cb_tp_connect(uint64_t ctx, uint32_t qpn, const CbTpAddr* remote);
int cb_tp_destroy_qp(uint64_t ctx, uint32_t qpn);

int cb_tp_post_send(uint64_t ctx, uint32_t qpn, const CbTpSendWr* wr);
int cb_tp_post_recv(uint64_t ctx, uint32_t qpn, uint64_t wr_id, const CbTpSge* sge, int num_sge);
int cb_tp_post_srq_recv(uint64_t ctx, uint32_t srq, uint64_t wr_id, const CbTpSge* sge, int num_sge);
// Polls up to `max` completions, waiting up to `timeout_us` for the first one.
// Returns the number of completions, or -1 when the queue is in error.
int cb_tp_poll_cq(uint64_t ctx, uint32_t cq, CbTpCompletion* out, int max, int64_t timeout_us);

// --- asynchronous events -----------------------------------------------------------------
// Waits up to `timeout_ms` for an event; returns 1 and fills the fields, 0 on time-out.
// Every delivered event must be acknowledged before the object it names can be destroyed.
int cb_tp_get_async_event(uint64_t ctx, int timeout_ms, int* event, uint32_t* object);
int cb_tp_ack_async_event(uint64_t ctx);

#ifdef __cplusplus
}
#endif
