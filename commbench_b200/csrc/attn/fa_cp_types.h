// Parameter block of the context-parallel attention kernel (fa_cp.cuh): what the planners
// (ring.cu, ulysses.cu) fill in and the kernel reads.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace cb {

static constexpr int CP_BM = 128;
static constexpr int CP_BN = 128;
static constexpr int CP_D = 128;
static constexpr int CP_SUB = 16384;
static constexpr int CP_TILE = 2 * CP_SUB;
static constexpr int CP_KST = 3, CP_VST = 2;
static constexpr int CP_SMEM = (2 + CP_KST + CP_VST) * CP_TILE + 1024;  // Q | K ring | V ring
static constexpr int CP_THREADS = 384;  // 4 utility warps (producer, MMA, 2 idle) + 8 softmax warps
static constexpr float CP_RESCALE_THRESHOLD = 8.f;
static constexpr int CP_MAX_SEGS = 32;
static constexpr int CP_MAX_QSEGS = 8;

struct CpSeg {   // keys row0 .. row0+nkeys-1 of the local K / V buffers (per batch)
  int row0;      // first row inside one batch of the buffer
  int kpos0;     // global sequence position of the first key
  int nkeys;
  int flag;      // index of the "ready" counter to wait for, or -1
};
struct CpQSeg {  // queries row0 .. row0+nrows-1 of one query tensor (per batch)
  int map;       // index into the tensor-map array, or -1 for the by-value local map
  int row0;
  int qpos0;     // global sequence position of the first query
  int nrows;
  int out;       // index into o[] / lse[]
  int pad;
};
struct CpCopy {  // 2-D piece pulled by the communication CTAs
  const uint8_t* src;
  uint8_t* dst;
  long long src_pitch, dst_pitch;
  int row_bytes;  // multiple of 16
  int nrows;
  int flag;       // counter bumped by every communication CTA when its share is stored
  int pad;
};

struct FaCpParams {
  CUtensorMap tm_k, tm_v;       // local buffers [rows, kv heads, 128]
  CUtensorMap tm_q_local;       // query map used by segments with map == -1
  const CUtensorMap* tm_q_arr;  // device array for the other query segments (may be null)
  CpSeg seg[CP_MAX_SEGS];
  CpQSeg qseg[CP_MAX_QSEGS];
  __nv_bfloat16* o[CP_MAX_QSEGS];  // [B, rows, o_heads, 128] per output tensor
  float* lse[CP_MAX_QSEGS];        // [B, o_heads, rows] or null
  int o_rows[CP_MAX_QSEGS];        // rows per batch of each output tensor
  int nseg, nqseg;
  int B;
  int heads;        // query heads handled by this launch
  int q_head0;      // first of them inside the query tensors
  int o_heads;      // heads of the output tensors
  int o_head0;      // first head written there
  int kv_group;     // query heads per key/value head
  int q_bstride;    // rows per batch in the query tensors
  int kv_bstride;   // rows per batch in the local K / V buffers
  int causal;
  float scale_log2;
  const CpCopy* copies;
  int ncopy, num_comm;
  uint32_t* flags;       // local counters
  uint32_t flag_target;  // a segment is ready when its counter has reached this value
  uint32_t* sched;       // [0] ticket counter, [1] CTAs that left
  uint32_t* status;
  unsigned long long timeout_ns;
};

}  // namespace cb
