"""Context-parallel attention: the local tcgen05 flash-attention forward, ring attention
(K/V chunks pulled from their owners while the previous chunk is being attended to) and
Ulysses attention (sequence<->head all-to-all around a full-sequence local attention).

Tensors are ``[B, S, H, D]`` bf16 with D = 128 (the layout the Ulysses exchange produces,
so no transposes are needed anywhere); GQA through ``Hq % Hkv == 0``.

The reference ships the communication halves only: the ring K/V rotation
(datasets/example057_thunderkitten_ring_attn_easy/nv/empty_thunderkitten_ring_attn.cu:97-134,
schedule :336-379) and the four Ulysses all-to-alls (datasets/example058_thunderkitten_ulysses_attn_easy/
nv/empty_thunderkitten_ulysses_attn.cu:330-359); the attention math, the exact merge of
partial results and causal load balancing are added here.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from ..config import get_config

from .. import _native as N
from ..runtime.context import CommContext, CommError, tensor_from_ptr
from ..utils.tracing import traced
from . import collectives as coll


@traced("cb200.flash_attention")
def flash_attention(q, k, v, causal: bool = True, q_offset: int = 0, kv_offset: int = 0,
                    scale: float | None = None, out=None, lse=None, status_ptr: int = 0,
                    stream=None, impl: int | None = None):
    """One key/value chunk: returns (o [B,Sq,Hq,D] bf16 normalised, lse [B,Hq,Sq] fp32).

    ``impl`` selects the kernel (default from ``CB200_ATTN_IMPL``): 4 = two query tiles per
    CTA with a softmax warp-group each, O and P in tensor memory (the product kernel);
    1 = the first design (one tile, O in registers), kept as a simple cross-check.

    ``q_offset`` / ``kv_offset`` are the global sequence positions of the first query / key;
    with ``causal`` key j is visible to query i iff kv_offset + j <= q_offset + i."""
    lib = N.load()
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        if not (t.is_cuda and t.is_contiguous() and t.dtype == torch.bfloat16 and t.dim() == 4
                and t.shape[-1] == 128):
            raise CommError(f"{n} must be a contiguous bf16 CUDA tensor [B, S, H, 128]")
    B, Sq, Hq, D = q.shape
    _, Skv, Hkv, _ = k.shape
    if v.shape != k.shape or k.shape[0] != B:
        raise CommError("k and v must have the same shape and q's batch size")
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device=q.device)
    sc = scale if scale is not None else 1.0 / math.sqrt(D)
    if impl is None:
        impl = get_config().attn_impl
    fn = {1: lib.cb_attn_fwd, 4: lib.cb_attn_fwd4}.get(impl)
    if fn is None:
        raise CommError(f"unknown attention kernel {impl} (1 or 4)")
    rc = fn(N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(out), N.ptr(lse), B, Sq, Skv, Hq, Hkv,
            q_offset, kv_offset, int(causal), C.c_float(sc), C.c_void_p(status_ptr),
            N.stream_ptr(stream))
    if rc != 0:
        raise CommError(f"attention launch failed: {N.last_error()}")
    return out, lse


def attn_merge(o_acc, lse_acc, o_part, lse_part, first: bool, stream=None):
    """acc <- exact merge of acc and a partial result over a disjoint key set."""
    lib = N.load()
    B, S, H, D = o_part.shape
    rc = lib.cb_attn_merge(N.ptr(o_acc), N.ptr(lse_acc), N.ptr(o_part), N.ptr(lse_part), B, S, H,
                           int(first), N.stream_ptr(stream))
    if rc != 0:
        raise CommError("attn_merge launch failed")


def zigzag_chunks(world: int, rank: int):
    """Causal load balancing: the sequence is cut into 2W chunks; rank r owns chunks r and
    2W-1-r, so every rank has the same amount of visible keys."""
    return rank, 2 * world - 1 - rank


class RingAttention:
    """Causal (or full) attention over a sequence sharded across ranks.

    Every rank publishes its K/V shard in symmetric memory.  Step i attends to the shard of
    rank (rank - i) mod W: the shard is pulled from its owner into a local double buffer by
    the copy engines on a side stream while the attention kernel works on the previous one,
    and partial results are merged exactly (running log-sum-exp).  With ``zigzag`` each rank
    holds two half-shards (chunks r and 2W-1-r of the sequence), which balances causal work.
    """

    def __init__(self, ctx: CommContext, batch: int, s_local: int, hq: int, hkv: int,
                 zigzag: bool = True):
        self.ctx, self.W, self.rank = ctx, ctx.world, ctx.rank
        self.B, self.Sl, self.Hq, self.Hkv = batch, s_local, hq, hkv
        self.zigzag = zigzag and ctx.world > 1
        if self.zigzag and s_local % 2:
            raise CommError("zigzag needs an even local sequence length")
        dev = ctx.device
        kv_bytes = batch * s_local * hkv * 128 * 2
        self.k_sym = ctx.alloc(kv_bytes)
        self.v_sym = ctx.alloc(kv_bytes)
        shape = (batch, s_local, hkv, 128)
        self.k_pub = self.k_sym.view(torch.bfloat16, shape)
        self.v_pub = self.v_sym.view(torch.bfloat16, shape)
        # peers' published shards as tensors over the peer mappings
        self.k_peer = [tensor_from_ptr(p, kv_bytes, dev, owner=ctx).view(torch.bfloat16).view(shape)
                       for p in self.k_sym.peer_ptrs]
        self.v_peer = [tensor_from_ptr(p, kv_bytes, dev, owner=ctx).view(torch.bfloat16).view(shape)
                       for p in self.v_sym.peer_ptrs]
        self.k_buf = [torch.empty(shape, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.v_buf = [torch.empty(shape, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.o_acc = torch.empty(batch, s_local, hq, 128, dtype=torch.float32, device=dev)
        self.lse_acc = torch.empty(batch, hq, s_local, dtype=torch.float32, device=dev)
        self.o_part = torch.empty(batch, s_local, hq, 128, dtype=torch.bfloat16, device=dev)
        self.lse_part = torch.empty(batch, hq, s_local, dtype=torch.float32, device=dev)
        self.copy_stream = torch.cuda.Stream(device=dev)
        self.launches = 0

    def _positions(self, r: int):
        """Global start positions of the (one or two) pieces of rank r's shard."""
        if not self.zigzag:
            return [(0, self.Sl, r * self.Sl)]
        h = self.Sl // 2
        a, b = zigzag_chunks(self.W, r)
        return [(0, h, a * h), (h, h, b * h)]

    @traced("cb200.ring_attention")
    def forward(self, q, k, v, causal: bool = True):
        ctx, W = self.ctx, self.W
        main = torch.cuda.current_stream()
        self.k_pub.copy_(k)
        self.v_pub.copy_(v)
        if W > 1:
            coll.barrier(ctx)            # everyone's shard is published
        first = True
        copied = [None, None]
        # prefetch of step 1
        def prefetch(step):
            src = (self.rank - step) % W
            buf = step & 1
            self.copy_stream.wait_stream(main)
            with torch.cuda.stream(self.copy_stream):
                self.k_buf[buf].copy_(self.k_peer[src], non_blocking=True)
                self.v_buf[buf].copy_(self.v_peer[src], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_stream)
            copied[buf] = ev
        if W > 1:
            prefetch(1)
        for step in range(W):
            src = (self.rank - step) % W
            if step == 0:
                kk, vv = self.k_pub, self.v_pub
            else:
                main.wait_event(copied[step & 1])
                kk, vv = self.k_buf[step & 1], self.v_buf[step & 1]
            for (q0, qn, qpos) in self._positions(self.rank):
                for (k0, kn, kpos) in self._positions(src):
                    if causal and kpos > qpos + qn - 1:
                        continue      # the whole key piece lies in the future of this query piece
                    qs = q[:, q0:q0 + qn]
                    if not qs.is_contiguous():
                        qs = qs.contiguous()
                    ks, vs = kk[:, k0:k0 + kn].contiguous(), vv[:, k0:k0 + kn].contiguous()
                    op = self.o_part[:, :qn].contiguous() if qn != self.Sl else self.o_part
                    lp = torch.empty(self.B, self.Hq, qn, dtype=torch.float32, device=q.device)
                    flash_attention(qs, ks, vs, causal=causal, q_offset=qpos, kv_offset=kpos,
                                    out=op, lse=lp, status_ptr=ctx.comm.status)
                    self.launches += 1
                    self._merge_piece(q0, qn, op, lp)
            if step + 2 <= W - 1:
                prefetch(step + 2)   # its buffer (step & 1) was consumed by the kernels above
        if W > 1:
            coll.barrier(ctx)            # nobody overwrites its published shard while it is read
        return self._finish(q)

    def _merge_piece(self, q0, qn, op, lp):
        if not hasattr(self, "_seen"):
            self._seen = set()
        key = q0
        firstp = key not in self._seen
        self._seen.add(key)
        if qn == self.Sl:
            attn_merge(self.o_acc, self.lse_acc, op, lp, firstp)
        else:
            # pieces are merged through contiguous temporaries (zigzag halves)
            oa = self.o_acc[:, q0:q0 + qn].contiguous() if not firstp else \
                torch.empty(self.B, qn, self.Hq, 128, dtype=torch.float32, device=op.device)
            la = self.lse_acc[:, :, q0:q0 + qn].contiguous() if not firstp else \
                torch.empty(self.B, self.Hq, qn, dtype=torch.float32, device=op.device)
            attn_merge(oa, la, op, lp, firstp)
            self.o_acc[:, q0:q0 + qn].copy_(oa)
            self.lse_acc[:, :, q0:q0 + qn].copy_(la)

    def _finish(self, q):
        self._seen = set()
        return self.o_acc.to(torch.bfloat16), self.lse_acc


@traced("cb200.ulysses_attention")
def ulysses_attention(ctx: CommContext, q, k, v, causal: bool = True):
    """Sequence-sharded in, sequence-sharded out: all-to-all q/k/v to head-sharded
    full-sequence tensors, local attention, all-to-all back (4 exchanges, as in the
    reference's Ulysses schedule)."""
    W = ctx.world
    if W == 1:
        return flash_attention(q, k, v, causal=causal, status_ptr=ctx.comm.status)[0]
    if q.shape[2] % W or k.shape[2] % W:
        raise CommError("Ulysses needs query and key/value heads divisible by the world size")
    qh = coll.all_to_all_4d(ctx, q, to_heads=True)
    kh = coll.all_to_all_4d(ctx, k, to_heads=True)
    vh = coll.all_to_all_4d(ctx, v, to_heads=True)
    oh, _ = flash_attention(qh, kh, vh, causal=causal, status_ptr=ctx.comm.status)
    return coll.all_to_all_4d(ctx, oh, to_heads=False)


def reference_attention(q, k, v, causal: bool = True, q_offset: int = 0, kv_offset: int = 0):
    """fp32 PyTorch reference with the same masking convention (returns o, lse)."""
    B, Sq, Hq, D = q.shape
    Hkv = k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    if causal:
        qi = torch.arange(Sq, device=q.device)[:, None] + q_offset
        kj = torch.arange(k.shape[1], device=q.device)[None, :] + kv_offset
        s = s.masked_fill(kj > qi, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.masked_fill(lse == float("-inf"), 0.0)[..., None])
    p = torch.nan_to_num(p, nan=0.0)
    o = (p @ vf).permute(0, 2, 1, 3)
    return o, lse
