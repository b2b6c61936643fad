// Ring attention as ONE kernel per rank: plan (segments, query halves, pieces to pull) and
// launch of the context-parallel attention kernel (fa_cp.cuh).
//
// Every rank keeps a key buffer and a value buffer [B][W slots][S_local][Hkv][128] in symmetric
// memory; slot r of rank r holds its own shard (the caller writes K / V there, or they are copied
// in), the other slots receive the peers' shards.  A launch pulls, in ring order
// rank-1, rank-2, ..., the shards this rank needs into their slots with a few communication
// CTAs (16-byte peer loads, local stores, one counter per shard piece) while the attention CTAs
// walk the same order - own shard first - with the running softmax state of a query tile kept
// in registers and tensor memory across all shards.  With the causal mask and zig-zag
// sharding (rank r owns chunks r and 2W-1-r of the sequence, so all ranks do the same amount
// of work) only the pieces that some local query can see are pulled.
//
// Reference (K/V rotation only, no attention): datasets/example057_thunderkitten_ring_attn_easy/
// nv/empty_thunderkitten_ring_attn.cu:97-134, stage schedule :336-379.
#include "cp_launch.h"

#include <cmath>
#include <string>
#include <vector>

#include "../prim/comm.h"
#include "../symm/driver_api.h"

using namespace cb;

extern "C" {

struct CbRingAttnDesc {
  int rank, world;
  int B, s_local, hq, hkv;
  int causal, zigzag;
  int num_comm;            // communication CTAs (0 when world == 1)
  float scale;
  const void* q;           // [B, S_local, Hq, 128] bf16, local
  void* o;                 // [B, S_local, Hq, 128] bf16, local
  void* lse;               // [B, Hq, S_local] fp32 or null
  void* k_slots[CB_MAX_RANKS];  // every rank's key buffer [B][W][S_local][Hkv][128]
  void* v_slots[CB_MAX_RANKS];
  void* flags;             // local uint32[64], zeroed once
  void* sched;             // local uint32[2], zeroed once
  void* copies;            // local device memory for the piece list (cb_ring_attn_copy_bytes())
  unsigned calls;          // launches made so far with these counters
  int write_plan;          // 1: (re)write the piece list (blocking copy; first call only)
  void* status;
  unsigned long long timeout_ns;
};

int cb_ring_attn_copy_bytes() { return static_cast<int>(sizeof(CpCopy)) * 4 * CB_MAX_RANKS * 8; }

// Global position of piece `pc` (0 or 1) of rank r's shard and its length.
static void ring_piece(const CbRingAttnDesc& d, int r, int pc, int* row0, int* pos0, int* n) {
  if (!d.zigzag) {
    *row0 = 0;
    *pos0 = r * d.s_local;
    *n = pc == 0 ? d.s_local : 0;
    return;
  }
  const int h = d.s_local / 2;
  *row0 = pc * h;
  *pos0 = (pc == 0 ? r : 2 * d.world - 1 - r) * h;
  *n = h;
}

int cb_ring_attn(const CbRingAttnDesc* dp, void* stream) {
  const CbRingAttnDesc& d = *dp;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int W = d.world, Sl = d.s_local;
  if (W < 1 || W > CB_MAX_RANKS || d.B < 1 || d.hq < 1 || d.hkv < 1 || d.hq % d.hkv != 0) {
    set_last_error("ring attention: bad shape (Hq must be a multiple of Hkv)");
    return -1;
  }
  if (Sl % (d.zigzag ? 512 : 256) != 0) {
    set_last_error("ring attention: the local sequence must be a multiple of 256 (512 with zig-zag)");
    return -1;
  }
  if (d.B * 4 * W > 4 * CB_MAX_RANKS * 8) {
    set_last_error("ring attention: batch too large for the piece list");
    return -1;
  }
  FaCpParams p = {};
  const int rows = d.B * W * Sl;
  if (cb_attn_make_tmap_bshd(&p.tm_k, d.k_slots[d.rank], rows, d.hkv)) return -1;
  if (cb_attn_make_tmap_bshd(&p.tm_v, d.v_slots[d.rank], rows, d.hkv)) return -1;
  if (cb_attn_make_tmap_bshd(&p.tm_q_local, d.q, d.B * Sl, d.hq)) return -1;
  p.tm_q_arr = nullptr;

  // The latest query position of this rank decides which pieces are visible at all.
  int q_max = 0;
  for (int pc = 0; pc < 2; ++pc) {
    int r0, p0, n;
    ring_piece(d, d.rank, pc, &r0, &p0, &n);
    if (n > 0 && p0 + n - 1 > q_max) q_max = p0 + n - 1;
  }
  // Segments in ring order (own shard, rank-1, ...) and the pieces to pull.
  std::vector<CpCopy> copies;
  const size_t row_bytes = static_cast<size_t>(d.hkv) * 256;
  int nflags = 0;
  for (int k = 0; k < W; ++k) {
    const int s = ((d.rank - k) % W + W) % W;
    for (int pc = 0; pc < 2; ++pc) {
      int r0, p0, n;
      ring_piece(d, s, pc, &r0, &p0, &n);
      if (n == 0) continue;
      if (d.causal && p0 > q_max) continue;  // no local query can see it
      if (p.nseg >= CP_MAX_SEGS) {
        set_last_error("ring attention: too many segments");
        return -1;
      }
      CpSeg& g = p.seg[p.nseg++];
      g.row0 = s * Sl + r0;
      g.kpos0 = p0;
      g.nkeys = n;
      g.flag = -1;
      if (s != d.rank) {
        g.flag = nflags++;
        for (int b = 0; b < d.B; ++b) {
          const size_t off = (static_cast<size_t>(b) * W * Sl + static_cast<size_t>(s) * Sl + r0) *
                             row_bytes;
          for (int kv = 0; kv < 2; ++kv) {
            CpCopy c = {};
            c.src = static_cast<const uint8_t*>(kv ? d.v_slots[s] : d.k_slots[s]) + off;
            c.dst = static_cast<uint8_t*>(kv ? d.v_slots[d.rank] : d.k_slots[d.rank]) + off;
            c.src_pitch = c.dst_pitch = 0;
            c.nrows = 1;
            const size_t bytes = static_cast<size_t>(n) * row_bytes;
            if (bytes > 0x7ffffff0ull) {
              set_last_error("ring attention: shard piece larger than 2 GB");
              return -1;
            }
            c.row_bytes = static_cast<int>(bytes);
            c.flag = g.flag;
            copies.push_back(c);
          }
        }
      }
    }
  }
  if (nflags > 64) {
    set_last_error("ring attention: too many counters");
    return -1;
  }
  // Query halves, late positions first (the long items under a causal mask).
  {
    int order[2] = {1, 0};
    for (int oi = 0; oi < 2; ++oi) {
      int r0, p0, n;
      ring_piece(d, d.rank, order[oi], &r0, &p0, &n);
      if (n == 0) continue;
      CpQSeg& q = p.qseg[p.nqseg++];
      q.map = -1;
      q.row0 = r0;
      q.qpos0 = p0;
      q.nrows = n;
      q.out = 0;
    }
  }
  p.o[0] = static_cast<__nv_bfloat16*>(d.o);
  p.lse[0] = static_cast<float*>(d.lse);
  p.o_rows[0] = Sl;
  p.B = d.B;
  p.heads = d.hq;
  p.q_head0 = 0;
  p.o_heads = d.hq;
  p.o_head0 = 0;
  p.kv_group = d.hq / d.hkv;
  p.q_bstride = Sl;
  p.kv_bstride = W * Sl;
  p.causal = d.causal;
  p.scale_log2 = d.scale * 1.4426950408889634f;
  p.copies = static_cast<const CpCopy*>(d.copies);
  p.ncopy = static_cast<int>(copies.size());
  p.num_comm = p.ncopy > 0 ? d.num_comm : 0;
  if (p.ncopy > 0 && p.num_comm < 1) {
    set_last_error("ring attention: world > 1 needs at least one communication CTA");
    return -1;
  }
  if (static_cast<int>(copies.size() * sizeof(CpCopy)) > cb_ring_attn_copy_bytes()) {
    set_last_error("ring attention: piece list too long");
    return -1;
  }
  p.flags = static_cast<uint32_t*>(d.flags);
  // every counter gets one increment per communication CTA for each of its 2 B pieces (K and V)
  p.flag_target = (d.calls + 1u) * static_cast<uint32_t>(2 * d.B * p.num_comm);
  p.sched = static_cast<uint32_t*>(d.sched);
  p.status = static_cast<uint32_t*>(d.status);
  p.timeout_ns = d.timeout_ns;
  if (d.write_plan && !copies.empty()) {
    cudaError_t e = cudaMemcpy(d.copies, copies.data(), copies.size() * sizeof(CpCopy),
                               cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      set_last_error(std::string("ring attention: piece list copy: ") + cudaGetErrorString(e));
      return -1;
    }
  }
  return cp_launch(p, p.num_comm + cp_num_items(p), st);
}

}  // extern "C"
