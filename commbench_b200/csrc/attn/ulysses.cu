// Ulysses attention as ONE kernel per rank, without stand-alone all-to-alls: plan and launch
// of the context-parallel attention kernel (fa_cp.cuh).
//
// Inputs are sequence-sharded [B, S_local, H, 128] tensors in symmetric memory.  Rank r attends,
// over the WHOLE sequence, for its slice of the heads (Hq/W query heads, Hkv/W key/value
// heads):
//   * the head slice of every rank's K and V shard is pulled into a local full-sequence buffer
//     [B][W S_local][Hkv/W][128] by a few communication CTAs, in sequence order, piece by piece
//     with a counter each (this is the K / V half of the sequence -> head exchange);
//   * Q tiles are fetched where they live: one 3-D tensor map per peer over its query tensor,
//     plain TMA loads of [128 rows, this head, 128] boxes (the Q exchange, fused into the load);
//   * O rows are stored straight into the owner's output tensor at this rank's head offset
//     (the head -> sequence exchange, fused into the epilogue).
// Cross-GPU barriers before (inputs published) and after (outputs complete, inputs free)
// bracket the launch.
//
// Reference (the four all-to-alls around an omitted attention):
// datasets/example058_thunderkitten_ulysses_attn_easy/nv/empty_thunderkitten_ulysses_attn.cu:59-120, :330-359.
#include "cp_launch.h"

#include <string>
#include <vector>

#include "../prim/comm.h"
#include "../symm/driver_api.h"

using namespace cb;

extern "C" {

struct CbUlyssesAttnDesc {
  int rank, world;
  int B, s_local, hq, hkv;   // full head counts; both divisible by world
  int causal;
  int num_comm;
  int pieces;                // readiness pieces per shard (world * pieces <= 32)
  float scale;
  void* q_peer[CB_MAX_RANKS];  // every rank's q [B, S_local, Hq, 128]
  void* k_peer[CB_MAX_RANKS];  // every rank's k [B, S_local, Hkv, 128]
  void* v_peer[CB_MAX_RANKS];
  void* o_peer[CB_MAX_RANKS];  // every rank's o [B, S_local, Hq, 128]
  void* kbuf;                  // local [B][W * S_local][Hkv / W][128]
  void* vbuf;
  void* qmaps;                 // local device memory, 64-byte aligned, W * 128 bytes
  void* flags;                 // local uint32[64], zeroed once
  void* sched;                 // local uint32[2], zeroed once
  void* copies;                // local device memory (cb_ulysses_attn_copy_bytes())
  unsigned calls;
  int write_plan;              // 1: (re)write tensor maps and piece list (blocking; first call)
  void* status;
  unsigned long long timeout_ns;
};

int cb_ulysses_attn_copy_bytes() { return static_cast<int>(sizeof(CpCopy)) * 2 * CP_MAX_SEGS * 8; }

int cb_ulysses_attn(const CbUlyssesAttnDesc* dp, void* stream) {
  const CbUlyssesAttnDesc& d = *dp;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int W = d.world, Sl = d.s_local;
  if (W < 1 || W > CB_MAX_RANKS || d.hq % W != 0 || d.hkv % W != 0 || d.hq % d.hkv != 0) {
    set_last_error("Ulysses attention: query and key/value heads must divide by the world size");
    return -1;
  }
  const int pieces = d.pieces < 1 ? 1 : d.pieces;
  if (Sl % (256 * pieces) != 0 || W * pieces > CP_MAX_SEGS) {
    set_last_error("Ulysses attention: S_local must be a multiple of 256 * pieces, W * pieces <= 32");
    return -1;
  }
  if (d.B * 2 * W * pieces > 2 * CP_MAX_SEGS * 8) {
    set_last_error("Ulysses attention: batch too large for the piece list");
    return -1;
  }
  const int hq_l = d.hq / W, hkv_l = d.hkv / W;
  FaCpParams p = {};
  const int S = W * Sl;
  if (cb_attn_make_tmap_bshd(&p.tm_k, d.kbuf, d.B * S, hkv_l)) return -1;
  if (cb_attn_make_tmap_bshd(&p.tm_v, d.vbuf, d.B * S, hkv_l)) return -1;
  p.tm_q_local = p.tm_k;  // unused: every query segment names a map of the array
  p.tm_q_arr = static_cast<const CUtensorMap*>(d.qmaps);
  if ((reinterpret_cast<uintptr_t>(d.qmaps) & 63u) != 0) {
    set_last_error("Ulysses attention: the tensor-map array must be 64-byte aligned");
    return -1;
  }
  std::vector<CpCopy> copies;
  const int piece_rows = Sl / pieces;
  for (int s = 0; s < W; ++s) {
    for (int pc = 0; pc < pieces; ++pc) {
      CpSeg& g = p.seg[p.nseg];
      g.row0 = s * Sl + pc * piece_rows;
      g.kpos0 = g.row0;
      g.nkeys = piece_rows;
      g.flag = p.nseg;
      ++p.nseg;
      for (int b = 0; b < d.B; ++b) {
        for (int kv = 0; kv < 2; ++kv) {
          CpCopy c = {};
          const uint8_t* src = static_cast<const uint8_t*>(kv ? d.v_peer[s] : d.k_peer[s]);
          uint8_t* dst = static_cast<uint8_t*>(kv ? d.vbuf : d.kbuf);
          c.src = src + ((static_cast<size_t>(b) * Sl + pc * piece_rows) * d.hkv +
                         static_cast<size_t>(d.rank) * hkv_l) * 256;
          c.dst = dst + (static_cast<size_t>(b) * S + g.row0) * hkv_l * 256;
          c.src_pitch = static_cast<long long>(d.hkv) * 256;
          c.dst_pitch = static_cast<long long>(hkv_l) * 256;
          c.row_bytes = hkv_l * 256;
          c.nrows = piece_rows;
          c.flag = g.flag;
          copies.push_back(c);
        }
      }
    }
  }
  // Query shards, late positions first.
  for (int s = W - 1; s >= 0; --s) {
    CpQSeg& q = p.qseg[p.nqseg++];
    q.map = s;
    q.row0 = 0;
    q.qpos0 = s * Sl;
    q.nrows = Sl;
    q.out = s;
    p.o[s] = static_cast<__nv_bfloat16*>(d.o_peer[s]);
    p.lse[s] = nullptr;
    p.o_rows[s] = Sl;
  }
  p.B = d.B;
  p.heads = hq_l;
  p.q_head0 = d.rank * hq_l;
  p.o_heads = d.hq;
  p.o_head0 = d.rank * hq_l;
  p.kv_group = hq_l / hkv_l;
  p.q_bstride = Sl;
  p.kv_bstride = S;
  p.causal = d.causal;
  p.scale_log2 = d.scale * 1.4426950408889634f;
  p.copies = static_cast<const CpCopy*>(d.copies);
  p.ncopy = static_cast<int>(copies.size());
  p.num_comm = d.num_comm < 1 ? 1 : d.num_comm;
  p.flags = static_cast<uint32_t*>(d.flags);
  p.flag_target = (d.calls + 1u) * static_cast<uint32_t>(2 * d.B * p.num_comm);
  p.sched = static_cast<uint32_t*>(d.sched);
  p.status = static_cast<uint32_t*>(d.status);
  p.timeout_ns = d.timeout_ns;
  if (d.write_plan) {
    std::vector<CUtensorMap> maps(W);
    for (int s = 0; s < W; ++s)
      if (cb_attn_make_tmap_bshd(&maps[s], d.q_peer[s], d.B * Sl, d.hq)) return -1;
    cudaError_t e = cudaMemcpy(d.qmaps, maps.data(), sizeof(CUtensorMap) * W, cudaMemcpyHostToDevice);
    if (e == cudaSuccess)
      e = cudaMemcpy(d.copies, copies.data(), copies.size() * sizeof(CpCopy),
                     cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      set_last_error(std::string("Ulysses attention: plan copy: ") + cudaGetErrorString(e));
      return -1;
    }
  }
  return cp_launch(p, p.num_comm + cp_num_items(p), st);
}

}  // extern "C"
