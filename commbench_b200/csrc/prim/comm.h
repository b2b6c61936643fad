// The communicator descriptor that every multi-GPU kernel receives by value.
//
// One process drives one GPU.  Each rank owns a *signal pad* (a small block of
// flag words inside symmetric memory); `pad[r]` is rank r's pad as mapped into
// this process (pad[rank] is local memory, the others go over NVLink).  When a
// multicast object could be bound, `mc_pad` aliases the pads of ALL ranks: a
// `multimem.red` to it updates every rank's copy inside the switch.
//
// Pad layout (uint32 words):
//   [0, CB_PAD_CHANNELS*8)            flag matrix: word [ch*8 + src] is written by rank `src`
//   [CB_PAD_NVLS_BASE, +CHANNELS)     counters bumped through the multicast alias
//   [CB_PAD_ABORT]                    non-zero once any rank gave up (peer-abort propagation)
//
// `epoch` holds one local counter per channel; a kernel that uses channel ch for
// k barriers reads e = epoch[ch], uses the values e+1 … e+k, and stores e+k back.
// All ranks launch the same kernels in the same order, so the counters stay in
// lock-step without the host being involved (CUDA-graph replay safe).
#pragma once
#include <stdint.h>

#include "status.h"

#define CB_PAD_CHANNELS 1024
#define CB_PAD_NVLS_BASE (CB_PAD_CHANNELS * CB_MAX_RANKS)
#define CB_PAD_ABORT (CB_PAD_NVLS_BASE + CB_PAD_CHANNELS)
#define CB_PAD_WORDS (CB_PAD_ABORT + 64)

struct CbComm {
  int32_t rank;
  int32_t world;
  uint32_t* pad[CB_MAX_RANKS];
  uint32_t* mc_pad;     // multicast alias of the pads, or nullptr
  uint32_t* epoch;      // [CB_PAD_CHANNELS] local device memory
  uint32_t* status;     // one word, host-mapped so the host can read it after a sync
  uint64_t timeout_ns;  // budget of every bounded wait
  // Debug stress: when non-zero every CTA of a collective kernel sleeps a pseudo-random time
  // below this many nanoseconds before it starts (a function of rank, CTA and call number), so
  // ordering assumptions that only hold when all CTAs start together show up in the tests.
  uint32_t jitter_ns;
  uint32_t reserved;
};
