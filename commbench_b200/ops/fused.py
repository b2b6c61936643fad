"""Fused tensor-parallel QK-RMSNorm (one kernel: partial sums, push all-reduce, scale, weight).

Reference counterpart: ``parallel_qknorm_across_head`` of
datasets/example101_sglang_qknorm_fused_easy/empty_sglang_qknorm_fused_easy.cu:132-209
(q_dim 6144, k_dim 1024 sharded over the ranks, 1...8192 tokens).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N
from ..runtime.context import CommError, EmuContext
from .tp import _Sym

_P8 = C.c_void_p * N.MAX_RANKS


class _QkArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("wq", C.c_void_p), ("wk", C.c_void_p),
        ("buf", _P8), ("seq", C.c_void_p),
        ("rank", C.c_int), ("world", C.c_int), ("tokens", C.c_int), ("max_tokens", C.c_int),
        ("q_local", C.c_int), ("k_local", C.c_int), ("eps", C.c_float),
        ("timeout_ns", C.c_ulonglong), ("status", C.c_void_p),
    ]


class TPQKNorm:
    """RMSNorm over the FULL q / k feature dimension when each rank holds a slice of it."""

    def __init__(self, ctx, max_tokens: int, q_local: int, k_local: int, eps: float = 1e-6):
        self.ctx, self.lib = ctx, ctx.lib
        self.emu = isinstance(ctx, EmuContext)
        self.W = ctx.world
        self.max_tokens, self.q_local, self.k_local, self.eps = max_tokens, q_local, k_local, eps
        self.buf = _Sym(ctx, 2 * max_tokens * self.W * 8, zero=True)
        n = self.W if self.emu else 1
        self.seq = [torch.zeros(4, dtype=torch.int32, device=ctx.device) for _ in range(n)]
        torch.cuda.synchronize(ctx.device)
        if not self.emu:
            ctx.host_barrier()
        assert self.lib.cb_sizeof_qknorm_args() == C.sizeof(_QkArgs)

    def _args(self, r, q, k, wq, wk) -> _QkArgs:
        a = _QkArgs()
        a.q, a.k, a.wq, a.wk = q.data_ptr(), k.data_ptr(), wq.data_ptr(), wk.data_ptr()
        for i in range(N.MAX_RANKS):
            a.buf[i] = self.buf.ptrs[i] if i < self.W else 0
        a.seq = self.seq[r if self.emu else 0].data_ptr()
        a.rank, a.world, a.tokens, a.max_tokens = r, self.W, q.shape[0], self.max_tokens
        a.q_local, a.k_local, a.eps = self.q_local, self.k_local, self.eps
        a.timeout_ns = self.ctx.timeout_ns
        a.status = self.ctx.comms[r].status if self.emu else self.ctx.comm.status
        return a

    def __call__(self, q, k, wq, wk, stream=None):
        """In place on q [tokens, q_local] and k [tokens, k_local] (lists in emulation)."""
        if self.emu:
            arr = (_QkArgs * self.W)(*[self._args(r, q[r], k[r], wq[r], wk[r])
                                       for r in range(self.W)])
            table = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(self.ctx.device)
            rc = self.lib.cb_qknorm(arr, self.W, C.c_void_p(table.data_ptr()), N.stream_ptr(stream))
            self._keep = table
        else:
            arr = (_QkArgs * 1)(self._args(self.ctx.rank, q, k, wq, wk))
            rc = self.lib.cb_qknorm(arr, 1, None, N.stream_ptr(stream))
        if rc != 0:
            raise CommError(f"qknorm failed: {N.last_error()}")
        return q, k


def reference_qknorm(q_parts, k_parts, wq_parts, wk_parts, eps: float):
    """fp32 reference: RMSNorm over the concatenation of all ranks' slices."""
    qf = torch.cat([t.float() for t in q_parts], dim=1)
    kf = torch.cat([t.float() for t in k_parts], dim=1)
    sq = torch.rsqrt(qf.pow(2).mean(dim=1, keepdim=True) + eps)
    sk = torch.rsqrt(kf.pow(2).mean(dim=1, keepdim=True) + eps)
    outs_q = [q.float() * sq * w.float() for q, w in zip(q_parts, wq_parts)]
    outs_k = [k.float() * sk * w.float() for k, w in zip(k_parts, wk_parts)]
    return outs_q, outs_k
