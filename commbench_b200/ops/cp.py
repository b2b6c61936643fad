"""Context-parallel attention: the local tcgen05 flash-attention forward, ring attention
(one kernel: communication CTAs pull the K/V shards in ring order while the other CTAs attend,
the softmax state of a query tile staying on chip across all shards) and Ulysses attention
(one kernel: K/V head slices pulled, Q tiles loaded from and O rows stored to their owners).

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


def zigzag_shard(x_full: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """The rows (dim 1) of a full-sequence tensor that rank ``rank`` owns under zig-zag sharding."""
    S = x_full.shape[1]
    h = S // (2 * world)
    a, b = zigzag_chunks(world, rank)
    return torch.cat([x_full[:, a * h:(a + 1) * h], x_full[:, b * h:(b + 1) * h]], dim=1).contiguous()


_P8 = C.c_void_p * N.MAX_RANKS


class _RingDesc(C.Structure):
    _fields_ = [
        ("rank", C.c_int), ("world", C.c_int), ("B", C.c_int), ("s_local", C.c_int),
        ("hq", C.c_int), ("hkv", C.c_int), ("causal", C.c_int), ("zigzag", C.c_int),
        ("num_comm", C.c_int), ("scale", C.c_float),
        ("q", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
        ("k_slots", _P8), ("v_slots", _P8),
        ("flags", C.c_void_p), ("sched", C.c_void_p), ("copies", C.c_void_p),
        ("calls", C.c_uint), ("write_plan", C.c_int),
        ("status", C.c_void_p), ("timeout_ns", C.c_ulonglong),
    ]


class _UlyssesDesc(C.Structure):
    _fields_ = [
        ("rank", C.c_int), ("world", C.c_int), ("B", C.c_int), ("s_local", C.c_int),
        ("hq", C.c_int), ("hkv", C.c_int), ("causal", C.c_int), ("num_comm", C.c_int),
        ("pieces", C.c_int), ("scale", C.c_float),
        ("q_peer", _P8), ("k_peer", _P8), ("v_peer", _P8), ("o_peer", _P8),
        ("kbuf", C.c_void_p), ("vbuf", C.c_void_p), ("qmaps", C.c_void_p),
        ("flags", C.c_void_p), ("sched", C.c_void_p), ("copies", C.c_void_p),
        ("calls", C.c_uint), ("write_plan", C.c_int),
        ("status", C.c_void_p), ("timeout_ns", C.c_ulonglong),
    ]


class _CpBase:
    """State shared by the two context-parallel attention ops: symmetric buffers seen the same
    way for real ranks and for virtual ranks on one GPU, the local counters of the kernel and
    the barriers around a launch."""

    def __init__(self, ctx):
        from ..runtime.context import EmuContext

        self.ctx = ctx
        self.lib = ctx.lib
        self.emu = isinstance(ctx, EmuContext)
        self.W = ctx.world
        self.nloc = self.W if self.emu else 1       # ranks driven by this process
        self.calls = 0
        self._plan_key = None

    def _ranks(self):
        return range(self.W) if self.emu else [self.ctx.rank]

    def _sym(self, nbytes):
        """(list of local tensors, one per rank driven here; list of W addresses)"""
        if self.emu:
            ts = self.ctx.alloc(nbytes)
            return ts, [t.data_ptr() for t in ts]
        blk = self.ctx.alloc(nbytes)
        return [blk.local], list(blk.peer_ptrs)

    def _local_state(self, copy_bytes):
        dev = self.ctx.device
        self.flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(self.nloc)]
        self.sched = [torch.zeros(4, dtype=torch.int32, device=dev) for _ in range(self.nloc)]
        self.copies = [torch.zeros(copy_bytes, dtype=torch.uint8, device=dev)
                       for _ in range(self.nloc)]

    def _status_ptr(self, i):
        return self.ctx.comms[i].status if self.emu else self.ctx.comm.status

    def _barrier(self):
        # Real ranks: a cross-GPU barrier kernel on the stream.  Virtual ranks run one after
        # the other on one stream, which orders them already.
        if not self.emu and self.W > 1:
            coll.barrier(self.ctx)


class RingAttention(_CpBase):
    """Causal (or full) attention over a sequence sharded across ranks, one kernel per call.

    Every rank owns a key and a value buffer ``[B, W, S_local, Hkv, 128]`` in symmetric memory;
    slot ``rank`` holds its own shard (``k_local`` / ``v_local`` are views of it: write K / V
    there and pass them to ``forward`` to avoid a copy).  The kernel's communication CTAs pull
    the shards this rank needs in ring order - rank-1, rank-2, ... - while its other CTAs attend,
    own shard first, keeping each query tile's running softmax state on chip across all
    shards.  ``zigzag`` (default): rank r holds chunks r and 2W-1-r of the sequence
    (:func:`zigzag_shard`), which balances causal work; with the causal mask only the pieces
    some local query can see are pulled at all.
    """

    def __init__(self, ctx, batch: int, s_local: int, hq: int, hkv: int, zigzag: bool = True,
                 num_comm: int | None = None):
        super().__init__(ctx)
        self.B, self.Sl, self.Hq, self.Hkv = batch, s_local, hq, hkv
        self.zigzag = bool(zigzag) and self.W > 1
        if s_local % (512 if self.zigzag else 256):
            raise CommError("ring attention: S_local must be a multiple of 256 (512 with zigzag)")
        self.num_comm = (num_comm if num_comm is not None else get_config().cp_comm_ctas) \
            if self.W > 1 else 0
        shape = (batch, self.W, s_local, hkv, 128)
        nbytes = batch * self.W * s_local * hkv * 256
        self.k_t, self.k_ptrs = self._sym(nbytes)
        self.v_t, self.v_ptrs = self._sym(nbytes)
        self.k_buf = [t[:nbytes].view(torch.bfloat16).view(shape) for t in self.k_t]
        self.v_buf = [t[:nbytes].view(torch.bfloat16).view(shape) for t in self.v_t]
        self._local_state(self.lib.cb_ring_attn_copy_bytes())
        torch.cuda.synchronize(ctx.device)
        if not self.emu:
            ctx.host_barrier()

    def k_local(self, i: int = 0) -> torch.Tensor:
        """This rank's own key slot, ``[B, S_local, Hkv, 128]`` (a view of symmetric memory)."""
        r = i if self.emu else self.ctx.rank
        return self.k_buf[i][:, r]

    def v_local(self, i: int = 0) -> torch.Tensor:
        r = i if self.emu else self.ctx.rank
        return self.v_buf[i][:, r]

    def _launch(self, i, r, q, o, lse, causal, scale, stream):
        d = _RingDesc()
        d.rank, d.world, d.B, d.s_local, d.hq, d.hkv = r, self.W, self.B, self.Sl, self.Hq, self.Hkv
        d.causal, d.zigzag, d.num_comm, d.scale = int(causal), int(self.zigzag), self.num_comm, scale
        d.q, d.o, d.lse = q.data_ptr(), o.data_ptr(), (lse.data_ptr() if lse is not None else 0)
        for x in range(N.MAX_RANKS):
            d.k_slots[x] = self.k_ptrs[x] if x < self.W else 0
            d.v_slots[x] = self.v_ptrs[x] if x < self.W else 0
        d.flags, d.sched = self.flags[i].data_ptr(), self.sched[i].data_ptr()
        d.copies = self.copies[i].data_ptr()
        d.calls = self.calls
        d.write_plan = int(self._plan_key != (bool(causal),))
        d.status, d.timeout_ns = self._status_ptr(i), self.ctx.timeout_ns
        if self.lib.cb_ring_attn(C.byref(d), N.stream_ptr(stream)) != 0:
            raise CommError(f"ring attention failed: {N.last_error()}")

    @traced("cb200.ring_attention")
    def forward(self, q, k, v, causal: bool = True, out=None, want_lse: bool = True,
                scale: float | None = None, stream=None):
        """``q`` [B, S_local, Hq, 128], ``k`` / ``v`` [B, S_local, Hkv, 128] bf16 (lists with one
        entry per virtual rank under an ``EmuContext``).  Returns ``(o, lse)``."""
        qs, ks, vs = (q, k, v) if self.emu else ([q], [k], [v])
        sc = scale if scale is not None else 1.0 / math.sqrt(128)
        outs, lses = [], []
        for i, _ in enumerate(self._ranks()):
            if ks[i].data_ptr() != self.k_local(i).data_ptr():
                self.k_local(i).copy_(ks[i])
            if vs[i].data_ptr() != self.v_local(i).data_ptr():
                self.v_local(i).copy_(vs[i])
        # A plan change (causal <-> full) rewrites the piece list and renumbers the counters:
        # nothing of the old plan may still run, and the counters start again from zero.
        if self._plan_key != (bool(causal),):
            torch.cuda.synchronize(self.ctx.device)
            for f in self.flags:
                f.zero_()
            self.calls = 0
        self._barrier()                       # every shard is published
        for i, r in enumerate(self._ranks()):
            qi = qs[i]
            if not (qi.is_contiguous() and qi.dtype == torch.bfloat16 and
                    tuple(qi.shape) == (self.B, self.Sl, self.Hq, 128)):
                raise CommError("q must be a contiguous bf16 tensor [B, S_local, Hq, 128]")
            o = (out[i] if self.emu else out) if out is not None else torch.empty_like(qi)
            lse = torch.empty(self.B, self.Hq, self.Sl, dtype=torch.float32, device=qi.device) \
                if want_lse else None
            self._launch(i, r, qi, o, lse, causal, sc, stream)
            outs.append(o)
            lses.append(lse)
        self._barrier()                       # nobody overwrites a shard that is still being read
        self._plan_key = (bool(causal),)
        self.calls += 1
        return (outs, lses) if self.emu else (outs[0], lses[0])


class UlyssesAttention(_CpBase):
    """Sequence-sharded in, sequence-sharded out attention where rank r attends for its slice
    of the heads over the whole sequence - in one kernel, without stand-alone all-to-alls: K / V
    head slices are pulled into a local full-sequence buffer by communication CTAs, Q tiles are
    TMA-loaded from their owners' memory, O rows are stored into their owners' outputs.

    ``q_buf`` / ``k_buf`` / ``v_buf`` / ``o_buf`` are this rank's tensors in symmetric memory;
    fill the inputs in place (or pass other tensors to ``forward``, which copies them in)."""

    def __init__(self, ctx, batch: int, s_local: int, hq: int, hkv: int,
                 num_comm: int | None = None, pieces: int | None = None):
        super().__init__(ctx)
        W = self.W
        if hq % W or hkv % W or hq % hkv:
            raise CommError("Ulysses needs query and key/value heads divisible by the world size")
        self.B, self.Sl, self.Hq, self.Hkv = batch, s_local, hq, hkv
        if pieces is None:
            pieces = max(1, min(4, 32 // W))
            while pieces > 1 and s_local % (256 * pieces):
                pieces //= 2
        if s_local % (256 * pieces):
            raise CommError("Ulysses attention: S_local must be a multiple of 256 * pieces")
        self.pieces = pieces
        self.num_comm = num_comm if num_comm is not None else get_config().cp_comm_ctas_ulysses
        qb, kb = batch * s_local * hq * 256, batch * s_local * hkv * 256
        self.q_t, self.q_ptrs = self._sym(qb)
        self.k_t, self.k_ptrs = self._sym(kb)
        self.v_t, self.v_ptrs = self._sym(kb)
        self.o_t, self.o_ptrs = self._sym(qb)
        qs, ks = (batch, s_local, hq, 128), (batch, s_local, hkv, 128)
        self.q_buf = [t[:qb].view(torch.bfloat16).view(qs) for t in self.q_t]
        self.k_buf = [t[:kb].view(torch.bfloat16).view(ks) for t in self.k_t]
        self.v_buf = [t[:kb].view(torch.bfloat16).view(ks) for t in self.v_t]
        self.o_buf = [t[:qb].view(torch.bfloat16).view(qs) for t in self.o_t]
        dev = ctx.device
        full = batch * W * s_local * (hkv // W) * 128
        self.kfull = [torch.empty(full, dtype=torch.bfloat16, device=dev) for _ in range(self.nloc)]
        self.vfull = [torch.empty(full, dtype=torch.bfloat16, device=dev) for _ in range(self.nloc)]
        self.qmaps = [torch.zeros(N.MAX_RANKS * 128, dtype=torch.uint8, device=dev)
                      for _ in range(self.nloc)]
        self._local_state(self.lib.cb_ulysses_attn_copy_bytes())
        torch.cuda.synchronize(dev)
        if not self.emu:
            ctx.host_barrier()

    def _launch(self, i, r, causal, scale, stream):
        d = _UlyssesDesc()
        d.rank, d.world, d.B, d.s_local, d.hq, d.hkv = r, self.W, self.B, self.Sl, self.Hq, self.Hkv
        d.causal, d.num_comm, d.pieces, d.scale = int(causal), self.num_comm, self.pieces, scale
        for x in range(N.MAX_RANKS):
            d.q_peer[x] = self.q_ptrs[x] if x < self.W else 0
            d.k_peer[x] = self.k_ptrs[x] if x < self.W else 0
            d.v_peer[x] = self.v_ptrs[x] if x < self.W else 0
            d.o_peer[x] = self.o_ptrs[x] if x < self.W else 0
        d.kbuf, d.vbuf = self.kfull[i].data_ptr(), self.vfull[i].data_ptr()
        d.qmaps = self.qmaps[i].data_ptr()
        d.flags, d.sched = self.flags[i].data_ptr(), self.sched[i].data_ptr()
        d.copies = self.copies[i].data_ptr()
        d.calls = self.calls
        d.write_plan = int(self._plan_key is None)
        d.status, d.timeout_ns = self._status_ptr(i), self.ctx.timeout_ns
        if self.lib.cb_ulysses_attn(C.byref(d), N.stream_ptr(stream)) != 0:
            raise CommError(f"Ulysses attention failed: {N.last_error()}")

    @traced("cb200.ulysses_attention")
    def forward(self, q=None, k=None, v=None, causal: bool = True, scale: float | None = None,
                stream=None):
        """Inputs that are not the op's own symmetric buffers are copied in; ``None`` means
        "already there".  Returns this rank's ``o_buf`` (valid until the next call)."""
        sc = scale if scale is not None else 1.0 / math.sqrt(128)
        for name, src, bufs in (("q", q, self.q_buf), ("k", k, self.k_buf), ("v", v, self.v_buf)):
            if src is None:
                continue
            srcs = src if self.emu else [src]
            for i, _ in enumerate(self._ranks()):
                if srcs[i].data_ptr() != bufs[i].data_ptr():
                    bufs[i].copy_(srcs[i])
        self._barrier()                       # inputs of every rank are in place
        for i, r in enumerate(self._ranks()):
            self._launch(i, r, causal, sc, stream)
        self._barrier()                       # every owner has all its output rows
        self._plan_key = True
        self.calls += 1
        return self.o_buf if self.emu else self.o_buf[0]


_ULYSSES_OPS: dict = {}


def ulysses_attention(ctx, q, k, v, causal: bool = True):
    """Functional form: keeps one :class:`UlyssesAttention` per (context, shape)."""
    from ..runtime.context import EmuContext

    q0 = q[0] if isinstance(ctx, EmuContext) else q
    k0 = k[0] if isinstance(ctx, EmuContext) else k
    key = (id(ctx), tuple(q0.shape), tuple(k0.shape))
    op = _ULYSSES_OPS.get(key)
    if op is None:
        op = UlyssesAttention(ctx, q0.shape[0], q0.shape[1], q0.shape[2], k0.shape[2])
        _ULYSSES_OPS[key] = op
    return op.forward(q, k, v, causal=causal)


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
