"""Expert-parallel MoE layer: router -> dispatch (fp8 payload, per-128-channel scales) ->
grouped GEMM (SwiGLU) -> grouped GEMM with the combine send fused into its epilogue ->
weighted combine reduction.

Per call and rank the kernels are (all from ``csrc/moe``):
  router_topk, moe_slots, [count all-gather], moe_plan, moe_sort_pairs, dispatch_send,
  recv_dequant, grouped_gemm(up; silu(gate) * up in its epilogue unless ``fused_swiglu`` is off,
  then a separate swiglu kernel), grouped_gemm(down, scatter), combine_reduce.
No host synchronisation happens between them: the receive side learns the row counts from
the all-gathered count matrix, never from the CPU (the reference's DeepEP path spins on
mapped host counters: datasets/example080_deepep_jit_dispatch_payload/nv/
empty_deepep_jit_dispatch_payload.cu:211-218).

Reference counterparts: ``deep_ep.ElasticBuffer.dispatch/combine``
(datasets/example080_deepep_jit_dispatch_payload/nv/build_and_run.py:679-759), the dispatch +
grouped GEMM of datasets/example056_thunderkitten_moe_dispatch_gemm_easy (same layer
constants H=7168, I=2048, 256 experts, top-8), the layout kernel of
datasets/example042_deepep_dispatch_layout.

With an :class:`~commbench_b200.runtime.context.EmuContext` the W ranks are virtual: every phase
is launched for all virtual ranks before the next phase starts, and no kernel of a phase
waits on a kernel of the same phase, so nothing ever waits on a later launch.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N
from ..runtime.context import CommError, EmuContext
from ..utils.tracing import traced
from . import collectives as coll

_P8 = C.c_void_p * N.MAX_RANKS


class _SendArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("topk_idx", C.c_void_p), ("topk_w", C.c_void_p),
        ("sorted_pair", C.c_void_p), ("src_pair_base", C.c_void_p), ("my_counts", C.c_void_p),
        ("send_row_base", C.c_void_p),
        ("recv_x", _P8), ("recv_scale", _P8), ("recv_meta", _P8), ("arrived", _P8),
        ("rank", C.c_int), ("world", C.c_int), ("T", C.c_int), ("K", C.c_int), ("H", C.c_int),
        ("E", C.c_int), ("max_rows", C.c_int), ("status", C.c_void_p), ("per_token", C.c_int),
    ]


class _RecvArgs(C.Structure):
    _fields_ = [
        ("recv_x", C.c_void_p), ("recv_scale", C.c_void_p), ("recv_meta", C.c_void_p),
        ("a_out", C.c_void_p), ("arrived", C.c_void_p), ("recv_expected", C.c_void_p),
        ("recv_base", C.c_void_p), ("H", C.c_int), ("max_rows", C.c_int),
        ("timeout_ns", C.c_ulonglong), ("status", C.c_void_p), ("ctas_done", C.c_void_p),
        ("per_token", C.c_int), ("T", C.c_int), ("K", C.c_int), ("stage_rows", C.c_int),
    ]


class _GroupedDesc(C.Structure):
    _fields_ = [
        ("max_rows", C.c_int), ("N", C.c_int), ("K", C.c_int), ("n_local_experts", C.c_int),
        ("down", C.c_int), ("rank", C.c_int), ("world", C.c_int), ("ctas", C.c_int),
        ("gated", C.c_int),
        ("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p),
        ("mblk_expert", C.c_void_p), ("n_mblocks", C.c_void_p), ("recv_meta", C.c_void_p),
        ("combine_peer", _P8), ("done_peer", _P8), ("done_ctas", C.c_void_p),
        ("status", C.c_void_p),
    ]


def router_topk(logits: torch.Tensor, k: int):
    """Softmax over experts, top-k, weights renormalised to sum to one (fp32 logits [T, E])."""
    lib = N.load()
    T, E = logits.shape
    logits = logits.float().contiguous()
    idx = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    N.check(lib.cb_moe_router_topk(N.ptr(logits), T, E, k, N.ptr(idx), N.ptr(w), N.stream_ptr()),
            "cb_moe_router_topk")
    return idx, w


def dispatch_layout(topk_idx: torch.Tensor, num_ranks: int, num_experts: int):
    """(num_tokens_per_expert[E], num_tokens_per_rank[R], is_token_in_rank[T,R])."""
    lib = N.load()
    T, K = topk_idx.shape
    idx = topk_idx.to(torch.int32).contiguous()
    per_e = torch.zeros(num_experts, dtype=torch.int32, device=idx.device)
    per_r = torch.zeros(num_ranks, dtype=torch.int32, device=idx.device)
    in_r = torch.zeros(T, num_ranks, dtype=torch.bool, device=idx.device)
    N.check(lib.cb_moe_dispatch_layout(N.ptr(idx), T, K, num_ranks, num_experts, N.ptr(per_e),
                                       N.ptr(per_r), N.ptr(in_r), N.stream_ptr()),
            "cb_moe_dispatch_layout")
    return per_e, per_r, in_r


def interleave_gate_up(w1: torch.Tensor, block: int = 128) -> torch.Tensor:
    """[E, 2I, H] with rows (gate | up) -> the same rows ordered per output block:
    gate rows j*block..(j+1)*block, then the up rows of the same outputs, for j = 0, 1, ...
    One 2*block-row tile of the product then holds both halves of `block` outputs, which is what
    the gated epilogue of the grouped GEMM combines into silu(gate) * up."""
    E, two_i, H = w1.shape
    I = two_i // 2
    if I % block:
        raise CommError(f"intermediate size must divide by {block}")
    g = w1[:, :I].reshape(E, I // block, 1, block, H)
    u = w1[:, I:].reshape(E, I // block, 1, block, H)
    return torch.cat([g, u], dim=2).reshape(E, two_i, H).contiguous()


class _RankState:
    """Buffers of one (virtual) rank."""

    def __init__(self, layer, r: int, dev):
        L = layer
        i32 = dict(dtype=torch.int32, device=dev)
        self.r = r
        self.slot = torch.empty(L.T * L.K, **i32)
        self.counts = torch.zeros(L.E, **i32)
        self.send_row_base = torch.empty(L.E, **i32)
        self.src_pair_base = torch.empty(L.E, **i32)
        self.recv_expected = torch.empty(L.El, **i32)
        self.recv_base = torch.empty(L.El + 1, **i32)
        self.mblk_expert = torch.zeros(L.max_rows // 128, **i32)
        self.n_mblocks = torch.zeros(1, **i32)
        self.n_rows = torch.zeros(1, **i32)
        self.sorted_pair = torch.empty(L.T * L.K, **i32)
        self.a = torch.empty(L.max_rows, L.H, dtype=torch.bfloat16, device=dev)
        self.h1 = None if L.fused_swiglu else \
            torch.empty(L.max_rows, 2 * L.I, dtype=torch.bfloat16, device=dev)
        self.s = torch.empty(L.max_rows, L.I, dtype=torch.bfloat16, device=dev)
        self.done_ctas = torch.zeros(4, **i32)
        self.recv_ctas = torch.zeros(L.El, **i32)      # CTAs of the receive kernel done, per expert
        self.y = torch.empty(L.T, L.H, dtype=torch.bfloat16, device=dev)
        g = torch.Generator(device=dev).manual_seed(L.seed * 977 + r)
        # bf16 expert weights N(0, 0.02): gate|up stacked [El, 2I, H] and down [El, H, I]
        self.w1 = (torch.randn(L.El, 2 * L.I, L.H, device=dev, generator=g) * 0.02).bfloat16()
        self.w2 = (torch.randn(L.El, L.H, L.I, device=dev, generator=g) * 0.02).bfloat16()
        # The gated up projection reads its own row order of the same weights (one more copy of w1).
        self.w1_gated = interleave_gate_up(self.w1) if L.fused_swiglu else None


class MoELayer:
    """Expert-parallel MoE feed-forward over `ctx` (real ranks or virtual ranks)."""

    def __init__(self, ctx, tokens: int, hidden: int, intermediate: int, num_experts: int,
                 topk: int, capacity_factor: float = 2.0, seed: int = 0,
                 fused_swiglu: bool | None = None, dispatch: str = "per_pair"):
        """``dispatch``: ``"per_pair"`` sends every (token, expert) selection as its own fp8 row,
        straight to its final position in the destination's per-expert buffer; ``"per_token"``
        sends a token once per destination RANK and lets the receive kernel expand it to the
        rows of that rank's experts (fewer NVLink bytes when a token selects several experts of
        one rank: about a third at top-8 over 8 ranks; the receive then waits for all of a
        rank's rows instead of expert by expert)."""
        self.ctx, self.lib = ctx, ctx.lib
        from ..config import get_config

        if dispatch not in ("per_pair", "per_token"):
            raise CommError("dispatch must be 'per_pair' or 'per_token'")
        self.per_token = dispatch == "per_token"
        if (self.lib.cb_sizeof_moe_send_args() != C.sizeof(_SendArgs)
                or self.lib.cb_sizeof_moe_recv_args() != C.sizeof(_RecvArgs)):
            raise CommError("MoE argument structs differ between the library and its Python mirror")

        self.fused_swiglu = get_config().moe_fused_swiglu if fused_swiglu is None else fused_swiglu
        self.emu = isinstance(ctx, EmuContext)
        self.W = ctx.world
        self.T, self.H, self.I, self.E, self.K = tokens, hidden, intermediate, num_experts, topk
        if num_experts % self.W or hidden % 256 or intermediate % 256 or (2 * intermediate) % 256:
            raise CommError("experts must divide by world; hidden and intermediate by 256")
        self.El = num_experts // self.W
        self.seed = seed
        avg = tokens * topk
        self.max_rows = (int(avg * capacity_factor) + self.El * 128 + 127) // 128 * 128
        dev = ctx.device
        from .tp import _Sym

        # rows of the fp8 receive buffer: the grouped layout, or one slot per (source rank, token)
        self.stage_rows = self.W * tokens if self.per_token else self.max_rows
        self.recv_x = _Sym(ctx, self.stage_rows * hidden)
        self.recv_scale = _Sym(ctx, self.stage_rows * (hidden // 128) * 4)
        self.recv_meta = _Sym(ctx, self.max_rows * 8)
        self.arrived = _Sym(ctx, max(self.El * 4, 64), zero=True)
        self.combine = _Sym(ctx, tokens * topk * hidden * 2)
        self.done = _Sym(ctx, 64, zero=True)
        self.states = [_RankState(self, r if self.emu else ctx.rank, dev)
                       for r in range(self.W if self.emu else 1)]
        self.sms = torch.cuda.get_device_properties(dev).multi_processor_count
        torch.cuda.synchronize(dev)
        if not self.emu:
            ctx.host_barrier()

    # ------------------------------------------------------------------ helpers
    def _status(self, st) -> int:
        return self.ctx.comms[st.r].status if self.emu else self.ctx.comm.status

    def _local(self, sym, st) -> torch.Tensor:
        return sym.tensors[st.r] if self.emu else sym.tensors[0]

    def weights(self, r: int = 0):
        st = self.states[r if self.emu else 0]
        return st.w1, st.w2

    # ------------------------------------------------------------------ stage timing
    def enable_stage_timing(self, on: bool = True):
        """Records a CUDA event after every stage of the next ``forward`` calls;
        ``stage_ms()`` (after a synchronize) returns the time spent in each stage."""
        self._marks = [] if on else None

    def _mark(self, name: str):
        if getattr(self, "_marks", None) is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._marks.append((name, ev))

    def stage_ms(self) -> dict:
        marks, out = getattr(self, "_marks", None) or [], {}
        for (_, e0), (name, e1) in zip(marks, marks[1:]):
            if name != "begin":
                out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        self._marks = []
        return out

    # ------------------------------------------------------------------ forward
    @traced("cb200.moe.forward")
    def forward(self, xs, topk_idx, topk_w, bias0=None, bias1=None):
        """xs [T, H] bf16, topk_idx [T, K] int32, topk_w [T, K] fp32 (lists in emulation).
        ``bias0`` / ``bias1``: optional [T, H] bf16 tensors added in the combine reduction (a
        shared expert's output, a residual).  Returns y [T, H] bf16 (list in emulation).

        The small kernels of the layer (slots, plan, pair sort, dispatch, receive, combine
        reduction) are chained with programmatic dependent launch: each may be scheduled while
        its predecessor still runs and waits on the device for it."""
        lib, W, E, K, T, H, I = self.lib, self.W, self.E, self.K, self.T, self.H, self.I
        if not self.emu:
            xs, topk_idx, topk_w = [xs], [topk_idx], [topk_w]
            bias0 = [bias0] if bias0 is not None else None
            bias1 = [bias1] if bias1 is not None else None
        sp = N.stream_ptr()
        n_pairs = T * K
        self._mark("begin")
        # 1. slots + counts
        for st, idx in zip(self.states, topk_idx):
            N.check(lib.cb_moe_slots(N.ptr(idx), n_pairs, E, N.ptr(st.slot), N.ptr(st.counts), sp),
                    "cb_moe_slots")
        # 2. count matrix on every rank
        if self.emu:
            counts_all = [torch.stack([s.counts for s in self.states]).contiguous()] * W
        else:
            counts_all = [coll.all_gather(self.ctx, self.states[0].counts.view(1, E)).contiguous()]
        self._mark("slots+count_gather")
        # 3. plan + sorted pairs (one launch)
        for st, idx, ca in zip(self.states, topk_idx, counts_all):
            N.check(lib.cb_moe_plan_sort(N.ptr(ca), W, E, st.r, N.ptr(idx), N.ptr(st.slot), n_pairs,
                                         N.ptr(st.sorted_pair), N.ptr(st.send_row_base),
                                         N.ptr(st.src_pair_base), N.ptr(st.recv_expected),
                                         N.ptr(st.recv_base), N.ptr(st.mblk_expert),
                                         N.ptr(st.n_mblocks), self.max_rows,
                                         C.c_void_p(self._status(st)), sp), "cb_moe_plan_sort")
        self._mark("plan+sort")
        # 4. dispatch push (quantise + send + per-expert arrival counters)
        for st, x, idx, w in zip(self.states, xs, topk_idx, topk_w):
            a = _SendArgs()
            a.x, a.topk_idx, a.topk_w = x.data_ptr(), idx.data_ptr(), w.data_ptr()
            a.sorted_pair, a.src_pair_base = st.sorted_pair.data_ptr(), st.src_pair_base.data_ptr()
            a.my_counts, a.send_row_base = st.counts.data_ptr(), st.send_row_base.data_ptr()
            for r in range(N.MAX_RANKS):
                ok = r < W
                a.recv_x[r] = self.recv_x.ptrs[r] if ok else 0
                a.recv_scale[r] = self.recv_scale.ptrs[r] if ok else 0
                a.recv_meta[r] = self.recv_meta.ptrs[r] if ok else 0
                a.arrived[r] = self.arrived.ptrs[r] if ok else 0
            a.rank, a.world, a.T, a.K, a.H, a.E, a.max_rows = st.r, W, T, K, H, E, self.max_rows
            a.status, a.per_token = self._status(st), int(self.per_token)
            N.check(lib.cb_moe_dispatch_send(C.byref(a), 4, sp), "cb_moe_dispatch_send")
        self._mark("dispatch_send")
        # 5. receive: wait per expert, dequantise to bf16, mark padding rows
        for st in self.states:
            ra = _RecvArgs()
            ra.recv_x = self._local(self.recv_x, st).data_ptr()
            ra.recv_scale = self._local(self.recv_scale, st).data_ptr()
            ra.recv_meta = self._local(self.recv_meta, st).data_ptr()
            ra.a_out = st.a.data_ptr()
            ra.arrived = self._local(self.arrived, st).data_ptr()
            ra.recv_expected, ra.recv_base = st.recv_expected.data_ptr(), st.recv_base.data_ptr()
            ra.H, ra.max_rows = H, self.max_rows
            ra.timeout_ns, ra.status = self.ctx.timeout_ns, self._status(st)
            ra.ctas_done = st.recv_ctas.data_ptr()    # the kernel re-arms the arrival counters
            ra.per_token, ra.T, ra.K, ra.stage_rows = int(self.per_token), T, K, self.stage_rows
            # about two CTAs per SM: the kernel streams max_rows * H bytes in and twice that out
            slices = max(4, -(-2 * self.sms // self.El))
            N.check(lib.cb_moe_recv_dequant(C.byref(ra), self.El, slices, sp), "cb_moe_recv_dequant")
        self._mark("recv_dequant")
        # 6. grouped GEMMs; the second one sends rows home
        for st in self.states:
            d = _GroupedDesc()
            d.max_rows, d.N, d.K, d.n_local_experts = self.max_rows, 2 * I, H, self.El
            d.down, d.rank, d.world, d.ctas = 0, st.r, W, self.sms
            if self.fused_swiglu:
                d.gated, d.a, d.b, d.c = 1, st.a.data_ptr(), st.w1_gated.data_ptr(), st.s.data_ptr()
            else:
                d.gated, d.a, d.b, d.c = 0, st.a.data_ptr(), st.w1.data_ptr(), st.h1.data_ptr()
            d.mblk_expert, d.n_mblocks = st.mblk_expert.data_ptr(), st.n_mblocks.data_ptr()
            d.status = self._status(st)
            N.check(lib.cb_moe_grouped_gemm(C.byref(d), sp), "grouped gemm (up)")
            self._mark("gemm_up")
            if not self.fused_swiglu:
                torch.mul(st.n_mblocks, 128, out=st.n_rows)
                N.check(lib.cb_moe_swiglu(N.ptr(st.h1), N.ptr(st.s), N.ptr(st.n_rows), I, sp),
                        "swiglu")
                self._mark("swiglu")
            d2 = _GroupedDesc()
            d2.max_rows, d2.N, d2.K, d2.n_local_experts = self.max_rows, H, I, self.El
            d2.down, d2.rank, d2.world, d2.ctas = 1, st.r, W, self.sms
            d2.a, d2.b, d2.c = st.s.data_ptr(), st.w2.data_ptr(), 0
            d2.mblk_expert, d2.n_mblocks = st.mblk_expert.data_ptr(), st.n_mblocks.data_ptr()
            d2.recv_meta = self._local(self.recv_meta, st).data_ptr()
            for r in range(N.MAX_RANKS):
                d2.combine_peer[r] = self.combine.ptrs[r] if r < W else 0
                d2.done_peer[r] = self.done.ptrs[r] if r < W else 0
            d2.done_ctas = st.done_ctas.data_ptr()
            d2.status = self._status(st)
            N.check(lib.cb_moe_grouped_gemm(C.byref(d2), sp), "grouped gemm (down)")
            self._mark("gemm_down+scatter")
        # 7. weighted reduction at the token owners
        for i, (st, idx, w) in enumerate(zip(self.states, topk_idx, topk_w)):
            N.check(lib.cb_moe_combine_reduce_bias(
                N.ptr(self._local(self.combine, st)), N.ptr(w), N.ptr(idx), N.ptr(st.y), T, K, H,
                N.ptr(self._local(self.done, st)), W, C.c_ulonglong(self.ctx.timeout_ns),
                C.c_void_p(self._status(st)), C.c_void_p(st.done_ctas.data_ptr() + 8),
                N.ptr(bias0[i] if bias0 is not None else None),
                N.ptr(bias1[i] if bias1 is not None else None), sp),
                "combine_reduce")
        self._mark("combine_reduce")
        ys = [st.y for st in self.states]
        return ys if self.emu else ys[0]

    @property
    def launches_per_call(self) -> int:
        # slots, count all-gather, plan+sort, dispatch, receive, two grouped GEMMs, combine
        # reduction; the unfused form adds the row count and the SwiGLU kernel
        return 8 if self.fused_swiglu else 10


def dispatch_rows(topk_idx: torch.Tensor, num_experts: int, world: int, per_token: bool) -> list[int]:
    """Token rows one rank sends to each destination rank for ``topk_idx`` [T, K] (negative =
    masked): one per selection (``per_token=False``) or one per distinct (token, rank) couple.
    Works on any device; the layer's NVLink payload is this times ``H + 4 * H / 128`` bytes."""
    per = num_experts // world
    idx = topk_idx.long()
    dst = torch.where(idx >= 0, idx // per, torch.full_like(idx, -1))          # [T, K]
    out = []
    for r in range(world):
        hit = dst == r
        out.append(int(hit.any(dim=1).sum()) if per_token else int(hit.sum()))
    return out


def expert_sort(topk_idx: torch.Tensor, num_experts: int):
    """Stable sort of the (token, k) selections by expert id.  Returns
    (sorted_pair [n] int32, counts [E] int32); masked (negative) selections are left out and
    the unused tail of ``sorted_pair`` is -1."""
    lib = N.load()
    idx = topk_idx.to(torch.int32).contiguous().view(-1)
    n = idx.numel()
    scratch = torch.empty(n + num_experts, dtype=torch.int32, device=idx.device)
    sorted_pair = torch.full((n,), -1, dtype=torch.int32, device=idx.device)
    counts = torch.empty(num_experts, dtype=torch.int32, device=idx.device)
    N.check(lib.cb_moe_expert_sort(N.ptr(idx), n, num_experts, N.ptr(scratch), N.ptr(sorted_pair),
                                   N.ptr(counts), N.stream_ptr()), "cb_moe_expert_sort")
    return sorted_pair, counts


def reference_moe(xs, topk_idx, topk_w, w1_all, w2_all, I: int):
    """Plain PyTorch fp32 reference of the whole layer for ONE source rank's tokens.
    `w1_all` [E, 2I, H], `w2_all` [E, H, I] (all experts).  Emulates the fp8 payload
    (per-128-channel scale, e4m3) and the bf16 roundings between the stages."""
    T, H = xs.shape
    xf = xs.float().view(T, H // 128, 128)
    amax = xf.abs().amax(dim=-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    xq = ((xf / scale).to(torch.float8_e4m3fn).float() * scale).view(T, H).bfloat16().float()
    y = torch.zeros(T, H, dtype=torch.float32, device=xs.device)
    K = topk_idx.shape[1]
    for k in range(K):
        e = topk_idx[:, k].long()
        for ex in e.unique().tolist():
            sel = (e == ex).nonzero().squeeze(1)
            h1 = (xq[sel] @ w1_all[ex].float().t()).bfloat16().float()
            s = (torch.nn.functional.silu(h1[:, :I]) * h1[:, I:]).bfloat16().float()
            o = (s @ w2_all[ex].float().t()).bfloat16().float()
            y[sel] += topk_w[sel, k:k + 1] * o
    return y
