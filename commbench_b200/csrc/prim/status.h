// Status words shared by host and device code.
//
// Every cross-GPU wait in this library is bounded.  When a wait runs out the
// kernel records ONE status word (first error wins) and returns; the host reads
// the word after the stream has drained and raises.  No kernel traps, asserts
// or spins without a limit.
//
// Layout of a status word:  [31:24] code  [23:16] phase  [15:0] detail
// (detail = peer rank, tile index or channel, whichever the phase documents).
#pragma once
#include <stdint.h>

#define CB_MAX_RANKS 8

enum CbStatusCode : uint32_t {
  CB_OK = 0,
  CB_TIMEOUT_PEER_FLAG = 1,   // a flag that a peer GPU should have written never arrived
  CB_TIMEOUT_MBARRIER = 2,    // an mbarrier inside one CTA never completed its phase
  CB_TIMEOUT_LOCAL_FLAG = 3,  // a flag another CTA of this GPU should have written never arrived
  CB_PEER_ABORT = 4,          // a peer published its abort word; this rank gave up too
  CB_BAD_ARGUMENT = 5,        // device-side argument check failed (bounds / alignment)
  CB_TIMEOUT_HOST_FLAG = 6,   // a flag the host (or a proxy thread) should have written never arrived
};

static inline uint32_t cb_make_status(uint32_t code, uint32_t phase, uint32_t detail) {
  return (code << 24) | ((phase & 0xffu) << 16) | (detail & 0xffffu);
}
static inline uint32_t cb_status_code(uint32_t s) { return s >> 24; }
static inline uint32_t cb_status_phase(uint32_t s) { return (s >> 16) & 0xffu; }
static inline uint32_t cb_status_detail(uint32_t s) { return s & 0xffffu; }

// Default wait budget: 2 s of %globaltimer.  Tests shorten it to exercise the
// time-out path (a flag that nothing sets) without harming the context.
#define CB_DEFAULT_TIMEOUT_NS 2000000000ull
