"""Collectives on symmetric memory: all_reduce / all_gather / reduce_scatter /
all_to_all (flat and 4-D Ulysses layouts) / broadcast / barrier.

Each op is ONE kernel launch of ``csrc/coll/collectives.cu``.  The PyTorch-facing
functions take a :class:`~commbench_b200.runtime.context.CommContext` (real ranks) or an
:class:`~commbench_b200.runtime.context.EmuContext` (virtual ranks on one GPU; tensors are
then lists with one entry per virtual rank).

Algorithm selection for all_reduce follows message size, like vLLM's custom
all-reduce (one-shot below a threshold, two-shot above:
datasets/example097_vllm_custom_all_reduce/nv/empty_vllm_custom_all_reduce.py:104-145) plus the
NVLS path of datasets/example048_thunderkitten_all_reduce_easy/nv/
empty_thunderkitten_all_reduce.cu:64-94 when a multicast object is bound.

**Ordering rule.**  The collectives of one context share the signal pad's channels (every
kernel uses channels 0 .. blocks-1 and their epoch counters) and the staging block
``coll_stage``.  They must therefore be *stream-ordered*: issue them on one stream, or order
the streams with events, so that no two collectives of the same context overlap on the
GPU - and every rank must issue them in the same order.  Overlapping calls race on the epochs
and on the staging buffer (wrong sums, or waits that run out after the time-out).  Use a
second ``CommContext`` for a second, concurrent stream of collectives.

**After a time-out.**  A wait that runs out records the context's status word and later waits
give up quickly, so results are garbage from then on.  Every launch first reads the
host-mapped status word (no synchronisation) and raises :class:`CommError` instead of
launching when it is set; ``ctx.check_status()`` reports and clears it, and
``ctx.reset_sync_state()`` re-arms the flags once every rank has stopped.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N
from ..config import get_config
from . import tuning
from ..runtime.context import CommContext, CommError, EmuContext

_DT = {torch.bfloat16: N.DT_BF16, torch.float16: N.DT_F16, torch.float32: N.DT_F32}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise CommError(f"dtype {t.dtype} not supported by the reducing collectives "
                        "(bf16, fp16, fp32)") from None


def _check_local(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise CommError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise CommError(f"{name} must be contiguous")
    if t.data_ptr() % 16 != 0:
        raise CommError(f"{name} must be 16-byte aligned")


def pick_blocks(nbytes: int, max_blocks: int, grain: int = 1 << 16) -> int:
    """One CTA per ``grain`` bytes of message (64 KiB by default), at least 1, at most
    ``max_blocks``."""
    return max(1, min(max_blocks, (nbytes + grain - 1) // grain))


def _default_cap(cfg, nbytes: int) -> int:
    """Grid cap of the bandwidth-bound collectives: one wave of 64 CTAs keeps the barrier cheap
    for small and medium messages; from 16 MB per rank up every SM takes part."""
    return cfg.coll_max_blocks_large if nbytes >= (16 << 20) else cfg.coll_max_blocks


def choose_all_reduce_algo(nbytes: int, world: int, has_multicast: bool) -> str:
    """Measured on 8xB200: the in-switch reduction wins at every size from 4 KB (16 us against
    27-31 us one-shot) to 1 GB (839 GB/s bus against 342 two-shot, 725 NCCL).  With two ranks
    the switch has nothing to save on large messages and the two-shot kernel is ahead from
    ~8 MB up."""
    cfg = get_config()
    if world == 1:
        return "oneshot"
    if has_multicast and nbytes >= cfg.ar_nvls_min_bytes and nbytes % 16 == 0 and \
            (world > 2 or nbytes < cfg.ar_nvls_max_bytes_two_ranks):
        return "nvls"
    if nbytes <= cfg.ar_oneshot_max_bytes:
        return "oneshot"
    return "twoshot"


def plan_all_reduce(ctx, nbytes: int, symmetric: bool) -> dict:
    """What ``all_reduce(..., algo="auto")`` will run for this message: ``{"algo", "blocks",
    "unroll"}`` (``blocks`` / ``unroll`` None where the size rule decides).  The measured table
    wins where it has a row; a row that asks for NVLS without a bound multicast object (or for a
    size that is not a multiple of 16 bytes) falls back to the size rule."""
    row = tuning.lookup("all_reduce", ctx.world, nbytes, "symmetric" if symmetric else "staged")
    algo = row.get("algo") or choose_all_reduce_algo(nbytes, ctx.world, ctx.has_multicast)
    if algo == "nvls" and not (ctx.has_multicast and nbytes % 16 == 0):
        return {"algo": choose_all_reduce_algo(nbytes, ctx.world, False), "blocks": None,
                "unroll": None}
    return {"algo": algo, "blocks": row.get("blocks"), "unroll": row.get("unroll")}


def _fill_args(comm: N.CbComm, sym_ptrs, mc_ptr, inp_ptr, out_ptr, nbytes, *, copy_in=0,
               copy_out=0, root=0, dtype=0, a2a=(0, 0, 0, 0, 0), unroll=0,
               variant=0) -> N.CollArgs:
    a = N.CollArgs()
    a.comm = comm
    for r in range(N.MAX_RANKS):
        a.sym[r] = sym_ptrs[r] if r < len(sym_ptrs) else 0
    a.mc = mc_ptr
    a.inp = inp_ptr
    a.out = out_ptr
    a.nbytes = nbytes
    a.copy_in, a.copy_out, a.root, a.dtype = copy_in, copy_out, root, dtype
    a.a2a_b, a.a2a_s_local, a.a2a_h, a.a2a_d, a.a2a_to_heads = a2a
    a.unroll, a.variant = int(unroll or 0), int(variant)
    return a


_OP_NAMES = ("all_reduce.oneshot", "all_reduce.twoshot", "all_reduce.nvls", "all_gather.pull",
             "all_gather.push", "reduce_scatter", "all_to_all", "all_to_all_4d", "broadcast")


def _refuse_after_failure(ctx):
    w = ctx.status_word()
    if w != 0:
        raise CommError(
            f"rank {ctx.rank}: an earlier kernel of this context reported "
            f"'{N.decode_status(w)}'; not launching on top of it - call ctx.check_status() / "
            "ctx.reset_sync_state() on every rank first")


def _launch(ctx, op: int, args: N.CollArgs, blocks: int, stream=None):
    _refuse_after_failure(ctx)
    if get_config().nvtx:
        from ..utils.tracing import nvtx_range

        with nvtx_range(f"cb200.{_OP_NAMES[op]}[{args.nbytes}B x{blocks}]"):
            rc = ctx.lib.cb_coll_launch(op, C.byref(args), None, 0, blocks, N.stream_ptr(stream))
    else:
        rc = ctx.lib.cb_coll_launch(op, C.byref(args), None, 0, blocks, N.stream_ptr(stream))
    if rc != 0:
        raise CommError(f"collective launch failed (rc={rc}): {N.last_error()}")


def _launch_emu(ctx: EmuContext, op: int, per_rank: list[N.CollArgs], blocks: int):
    table = ctx.args_table(per_rank)
    rc = ctx.lib.cb_coll_launch(op, C.byref(per_rank[0]), C.c_void_p(table.data_ptr()), ctx.world,
                                blocks, N.stream_ptr())
    if rc != 0:
        raise CommError(f"emulated collective launch failed (rc={rc}): {N.last_error()}")
    ctx._keepalive = table  # until the stream has consumed it


def _pad16(n: int) -> int:
    return (n + 15) // 16 * 16


# =============================================================== real contexts
def all_reduce(ctx: CommContext, x: torch.Tensor, out: torch.Tensor | None = None,
               algo: str = "auto", max_blocks: int | None = None, stream=None,
               blocks: int | None = None, unroll: int | None = None) -> torch.Tensor:
    """Sum over ranks.  In place when ``out`` is None.  ``algo`` in
    {"auto", "oneshot", "twoshot", "twoshot_push", "nvls"}; "auto" takes the measured table
    (:mod:`.tuning`) where it has a row and the size rule of :func:`choose_all_reduce_algo`
    otherwise.  ``blocks`` / ``unroll`` force the grid size and the 16-byte vectors each
    thread keeps in flight."""
    _check_local(x, "x")
    out = x if out is None else out
    _check_local(out, "out")
    nbytes = x.numel() * x.element_size()
    if nbytes == 0:
        return out
    cfg = get_config()
    sym = ctx.find_block(x) if nbytes % 16 == 0 else None
    if algo == "auto":
        plan = plan_all_reduce(ctx, nbytes, sym is not None)
        algo = plan["algo"]
        if blocks is None and max_blocks is None:
            blocks = plan["blocks"]
        if unroll is None:
            unroll = plan["unroll"]
    if algo == "nvls" and not ctx.has_multicast:
        raise CommError("algo='nvls' needs a bound multicast object (not available here)")
    if algo not in ("oneshot", "twoshot", "twoshot_push", "nvls"):
        raise CommError(f"unknown all-reduce algorithm {algo!r}")
    if blocks is None:
        # One-shot is latency bound: every CTA reads its slice from all W ranks, so slices are
        # kept small; the chunked algorithms move nbytes / W per rank.
        grain = cfg.ar_oneshot_grain_bytes if algo == "oneshot" else cfg.ar_chunk_grain_bytes
        cap = max_blocks or cfg.coll_max_blocks
        if max_blocks is None and algo.startswith("twoshot") and nbytes >= (16 << 20):
            cap = cfg.coll_max_blocks_large      # pull-based: more loads in flight pay off
        blocks = pick_blocks(nbytes, cap, grain)
    dt = _dtype_code(x)
    if algo == "oneshot":
        # Result must not land in memory peers read: stage unless x is symmetric and out is not x.
        if sym is not None and out.data_ptr() != x.data_ptr():
            a = _fill_args(ctx.comm, sym[0], sym[1], x.data_ptr(), out.data_ptr(), nbytes, dtype=dt)
        else:
            st = ctx.named("coll_stage", _pad16(nbytes))
            a = _fill_args(ctx.comm, st.peer_ptrs, st.mc_ptr, x.data_ptr(), out.data_ptr(), nbytes,
                           copy_in=1, dtype=dt)
        _launch(ctx, N.OP_AR_ONESHOT, a, blocks, stream)
        return out
    op = N.OP_AR_NVLS if algo == "nvls" else N.OP_AR_TWOSHOT
    var = 1 if algo == "twoshot_push" else 0
    if sym is not None and (algo != "nvls" or sym[1]):
        same = out.data_ptr() == x.data_ptr()
        a = _fill_args(ctx.comm, sym[0], sym[1], x.data_ptr(), out.data_ptr(), nbytes,
                       copy_in=0, copy_out=0 if same else 1, dtype=dt, unroll=unroll, variant=var)
    else:
        st = ctx.named("coll_stage", _pad16(nbytes))
        a = _fill_args(ctx.comm, st.peer_ptrs, st.mc_ptr, x.data_ptr(), out.data_ptr(), nbytes,
                       copy_in=1, copy_out=1, dtype=dt, unroll=unroll, variant=var)
    _launch(ctx, op, a, blocks, stream)
    return out


def all_gather(ctx: CommContext, x: torch.Tensor, out: torch.Tensor | None = None,
               max_blocks: int | None = None, stream=None, blocks: int | None = None,
               unroll: int | None = None, multicast: bool | None = None) -> torch.Tensor:
    """Concatenates every rank's ``x`` along dim 0.  If ``out`` lives in the symmetric heap the
    shards are pushed straight into every rank's copy (one multimem.st per vector when NVLS
    is bound); otherwise shards are staged and pulled."""
    _check_local(x, "x")
    nbytes = x.numel() * x.element_size()
    if out is None:
        out = torch.empty((ctx.world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype,
                          device=x.device)
    _check_local(out, "out")
    if out.numel() * out.element_size() != ctx.world * nbytes:
        raise CommError("all_gather: out has the wrong size")
    cfg = get_config()
    osym = ctx.find_block(out)
    push = osym is not None and nbytes % 16 == 0
    row = tuning.lookup("all_gather", ctx.world, nbytes, "push" if push else "pull")
    if blocks is None:
        blocks = (row.get("blocks") if max_blocks is None else None) or \
            pick_blocks(nbytes, max_blocks or _default_cap(cfg, nbytes))
    if unroll is None:
        unroll = row.get("unroll")
    if push:
        # One multicast store replaces W-1 peer stores; between two ranks it replaces one and
        # was measured slower than plain stores for large shards.
        use_mc = multicast if multicast is not None else row.get("multicast")
        if use_mc is None:
            use_mc = ctx.world > 2 or nbytes < cfg.ar_nvls_max_bytes_two_ranks
        mc = osym[1] if use_mc else 0
        a = _fill_args(ctx.comm, osym[0], mc, x.data_ptr(), out.data_ptr(), nbytes, unroll=unroll)
        _launch(ctx, N.OP_AG_PUSH, a, blocks, stream)
        return out
    xsym = ctx.find_block(x)
    if xsym is not None:
        a = _fill_args(ctx.comm, xsym[0], 0, x.data_ptr(), out.data_ptr(), nbytes, unroll=unroll)
    else:
        st = ctx.named("coll_stage", _pad16(nbytes))
        a = _fill_args(ctx.comm, st.peer_ptrs, 0, x.data_ptr(), out.data_ptr(), nbytes, copy_in=1,
                       unroll=unroll)
    _launch(ctx, N.OP_AG_PULL, a, blocks, stream)
    return out


def reduce_scatter(ctx: CommContext, x: torch.Tensor, out: torch.Tensor | None = None,
                   use_nvls: bool | None = None, max_blocks: int | None = None,
                   stream=None, blocks: int | None = None,
                   unroll: int | None = None) -> torch.Tensor:
    """``x`` holds W equal chunks along dim 0; rank r receives the sum of chunk r."""
    _check_local(x, "x")
    nbytes = x.numel() * x.element_size()
    if x.shape[0] % ctx.world != 0 or (nbytes // ctx.world) % 16 != 0:
        raise CommError("reduce_scatter: dim 0 must divide by world and chunks be 16-byte multiples")
    if out is None:
        out = torch.empty((x.shape[0] // ctx.world,) + tuple(x.shape[1:]), dtype=x.dtype,
                          device=x.device)
    _check_local(out, "out")
    cfg = get_config()
    dt = _dtype_code(x)
    sym = ctx.find_block(x)
    row = tuning.lookup("reduce_scatter", ctx.world, nbytes,
                        "symmetric" if sym is not None else "staged")
    if blocks is None:
        blocks = (row.get("blocks") if max_blocks is None else None) or \
            pick_blocks(nbytes // ctx.world, max_blocks or _default_cap(cfg, nbytes // ctx.world))
    if unroll is None:
        unroll = row.get("unroll")
    if use_nvls is None:
        use_nvls = row.get("nvls")
    if use_nvls is None:
        # Between two ranks the switch reduction adds a hop and saves no link bytes: above a few
        # MB plain peer loads are faster (measured), as for all-reduce.
        want_nvls = ctx.has_multicast and (ctx.world > 2 or nbytes < cfg.ar_nvls_max_bytes_two_ranks)
    else:
        want_nvls = use_nvls and ctx.has_multicast
    if sym is not None:
        a = _fill_args(ctx.comm, sym[0], sym[1] if want_nvls else 0, x.data_ptr(), out.data_ptr(),
                       nbytes, dtype=dt, unroll=unroll)
    else:
        st = ctx.named("coll_stage", nbytes)
        a = _fill_args(ctx.comm, st.peer_ptrs, st.mc_ptr if want_nvls else 0, x.data_ptr(),
                       out.data_ptr(), nbytes, copy_in=1, dtype=dt, unroll=unroll)
    _launch(ctx, N.OP_RS, a, blocks, stream)
    return out


def all_to_all(ctx: CommContext, x: torch.Tensor, out: torch.Tensor | None = None,
               max_blocks: int | None = None, stream=None, blocks: int | None = None,
               unroll: int | None = None, push: bool | None = None) -> torch.Tensor:
    """Flat exchange of W equal chunks along dim 0 (``all_to_all_single`` semantics).

    Pull form: every rank loads its chunk out of each peer's (symmetric or staged) input.
    Push form (``push=True``; the default when ``out`` lives in the symmetric heap): every rank
    stores chunk p of its local ``x`` straight into rank p's output - no staging copy, and
    stores need no request packet in the opposite direction."""
    _check_local(x, "x")
    nbytes = x.numel() * x.element_size()
    if x.shape[0] % ctx.world != 0 or (nbytes // ctx.world) % 16 != 0:
        raise CommError("all_to_all: dim 0 must divide by world and chunks be 16-byte multiples")
    out = torch.empty_like(x) if out is None else out
    _check_local(out, "out")
    cfg = get_config()
    sym = ctx.find_block(x)
    osym = ctx.find_block(out)
    kind = "out_symmetric" if osym is not None else ("symmetric" if sym is not None else "staged")
    row = tuning.lookup("all_to_all", ctx.world, nbytes, kind)
    if push is None:
        push = row.get("push")
    if push is None:
        push = osym is not None
    if blocks is None:
        blocks = (row.get("blocks") if max_blocks is None else None) or \
            pick_blocks(nbytes, max_blocks or _default_cap(cfg, nbytes))
    if unroll is None:
        unroll = row.get("unroll")
    if push:
        if osym is not None:
            a = _fill_args(ctx.comm, osym[0], 0, x.data_ptr(), out.data_ptr(), nbytes,
                           unroll=unroll, variant=1)
        else:
            st = ctx.named("coll_stage", nbytes)
            a = _fill_args(ctx.comm, st.peer_ptrs, 0, x.data_ptr(), out.data_ptr(), nbytes,
                           copy_out=1, unroll=unroll, variant=1)
    elif sym is not None:
        a = _fill_args(ctx.comm, sym[0], 0, x.data_ptr(), out.data_ptr(), nbytes, unroll=unroll)
    else:
        st = ctx.named("coll_stage", nbytes)
        a = _fill_args(ctx.comm, st.peer_ptrs, 0, x.data_ptr(), out.data_ptr(), nbytes, copy_in=1,
                       unroll=unroll)
    _launch(ctx, N.OP_A2A_FLAT, a, blocks, stream)
    return out


def all_to_all_4d(ctx: CommContext, x: torch.Tensor, to_heads: bool,
                  out: torch.Tensor | None = None, max_blocks: int | None = None,
                  stream=None) -> torch.Tensor:
    """Ulysses layouts.  ``to_heads``: [B, S/W, H, D] -> [B, S, H/W, D]; else the inverse
    ([B, S, H/W, D] -> [B, S/W, H, D]).  Same exchange as ``NcclAllToAll.Run`` with
    scatter_idx=2, gather_idx=1 (datasets/example020_torch_distributed_nccl_alltoall/
    empty_nccl_alltoall.py:67-89) and the TMA kernel of datasets/example049_thunderkitten_alltoall_easy/
    nv/empty_thunderkitten_alltoall.cu:60-121."""
    _check_local(x, "x")
    W = ctx.world
    if x.dim() != 4:
        raise CommError("all_to_all_4d expects a 4-D tensor")
    if to_heads:
        B, Sl, H, D = x.shape
        if H % W:
            raise CommError("heads must divide by world")
        oshape = (B, Sl * W, H // W, D)
    else:
        B, S, Hl, D = x.shape
        if S % W:
            raise CommError("sequence must divide by world")
        Sl, H = S // W, Hl * W
        oshape = (B, Sl, H, D)
    if (D * x.element_size()) % 16:
        raise CommError("head_dim * element size must be a multiple of 16 bytes")
    out = torch.empty(oshape, dtype=x.dtype, device=x.device) if out is None else out
    _check_local(out, "out")
    nbytes = x.numel() * x.element_size()
    cfg = get_config()
    blocks = pick_blocks(nbytes, max_blocks or _default_cap(cfg, nbytes))
    geo = (B, Sl, H, D, 1 if to_heads else 0)
    sym = ctx.find_block(x)
    if sym is not None:
        a = _fill_args(ctx.comm, sym[0], 0, x.data_ptr(), out.data_ptr(), nbytes, a2a=geo)
    else:
        st = ctx.named("coll_stage", nbytes)
        a = _fill_args(ctx.comm, st.peer_ptrs, 0, x.data_ptr(), out.data_ptr(), nbytes, copy_in=1,
                       a2a=geo)
    _launch(ctx, N.OP_A2A_4D, a, blocks, stream)
    return out


def broadcast(ctx: CommContext, x: torch.Tensor, root: int = 0, max_blocks: int | None = None,
              stream=None) -> torch.Tensor:
    """In-place broadcast of ``x`` from ``root``."""
    _check_local(x, "x")
    nbytes = x.numel() * x.element_size()
    cfg = get_config()
    blocks = pick_blocks(nbytes, max_blocks or _default_cap(cfg, nbytes))
    st = ctx.named("coll_stage", _pad16(nbytes))
    if ctx.has_multicast and x.data_ptr() % 16 == 0:
        a = _fill_args(ctx.comm, st.peer_ptrs, st.mc_ptr, x.data_ptr(), x.data_ptr(), nbytes,
                       copy_out=1, root=root)
    else:
        a = _fill_args(ctx.comm, st.peer_ptrs, 0, x.data_ptr(), x.data_ptr(), nbytes, copy_in=1,
                       root=root)
    _launch(ctx, N.OP_BCAST, a, blocks, stream)
    return x


def barrier(ctx: CommContext, iters: int = 1, use_nvls: bool = False, stream=None):
    """Device-side barrier across ranks (one <<<1,32>>> launch)."""
    if use_nvls and not ctx.has_multicast:
        raise CommError("NVLS barrier needs a bound multicast object")
    a = _fill_args(ctx.comm, [], 0, 0, 0, 0)
    rc = ctx.lib.cb_barrier_launch(C.byref(a), None, 0, iters, int(use_nvls), N.stream_ptr(stream))
    if rc != 0:
        raise CommError(f"barrier launch failed: {N.last_error()}")


# ============================================================ emulated contexts
def _emu_blocks(nbytes: int) -> int:
    return pick_blocks(nbytes, 8)


def emu_all_reduce(ctx: EmuContext, xs: list[torch.Tensor], algo: str = "oneshot",
                   blocks: int | None = None, unroll: int = 0) -> list[torch.Tensor]:
    W = ctx.world
    nbytes = xs[0].numel() * xs[0].element_size()
    stage = ctx.alloc(_pad16(nbytes))
    outs = [torch.empty_like(x) for x in xs]
    sym = [s.data_ptr() for s in stage]
    op = {"oneshot": N.OP_AR_ONESHOT, "twoshot": N.OP_AR_TWOSHOT,
          "twoshot_push": N.OP_AR_TWOSHOT}[algo]
    args = [_fill_args(ctx.comms[r], sym, 0, xs[r].data_ptr(), outs[r].data_ptr(), nbytes,
                       copy_in=1, copy_out=1, dtype=_dtype_code(xs[r]), unroll=unroll,
                       variant=1 if algo == "twoshot_push" else 0) for r in range(W)]
    _launch_emu(ctx, op, args, blocks or _emu_blocks(nbytes))
    ctx._stage = stage
    return outs


def emu_all_gather(ctx: EmuContext, xs: list[torch.Tensor], push: bool = False,
                   blocks: int | None = None, unroll: int = 0) -> list[torch.Tensor]:
    W = ctx.world
    nbytes = xs[0].numel() * xs[0].element_size()
    oshape = (W * xs[0].shape[0],) + tuple(xs[0].shape[1:])
    if push:
        outs_raw = ctx.alloc(W * nbytes)
        outs = [o[:W * nbytes].view(xs[0].dtype).view(oshape) for o in outs_raw]
        sym = [o.data_ptr() for o in outs_raw]
        args = [_fill_args(ctx.comms[r], sym, 0, xs[r].data_ptr(), outs[r].data_ptr(), nbytes,
                           unroll=unroll) for r in range(W)]
        _launch_emu(ctx, N.OP_AG_PUSH, args, blocks or _emu_blocks(nbytes))
        ctx._stage = outs_raw
        return outs
    stage = ctx.alloc(_pad16(nbytes))
    outs = [torch.empty(oshape, dtype=xs[0].dtype, device=xs[0].device) for _ in range(W)]
    sym = [s.data_ptr() for s in stage]
    args = [_fill_args(ctx.comms[r], sym, 0, xs[r].data_ptr(), outs[r].data_ptr(), nbytes,
                       copy_in=1, unroll=unroll) for r in range(W)]
    _launch_emu(ctx, N.OP_AG_PULL, args, blocks or _emu_blocks(nbytes))
    ctx._stage = stage
    return outs


def emu_reduce_scatter(ctx: EmuContext, xs: list[torch.Tensor],
                       blocks: int | None = None, unroll: int = 0) -> list[torch.Tensor]:
    W = ctx.world
    nbytes = xs[0].numel() * xs[0].element_size()
    stage = ctx.alloc(nbytes)
    oshape = (xs[0].shape[0] // W,) + tuple(xs[0].shape[1:])
    outs = [torch.empty(oshape, dtype=xs[0].dtype, device=xs[0].device) for _ in range(W)]
    sym = [s.data_ptr() for s in stage]
    args = [_fill_args(ctx.comms[r], sym, 0, xs[r].data_ptr(), outs[r].data_ptr(), nbytes,
                       copy_in=1, dtype=_dtype_code(xs[r]), unroll=unroll) for r in range(W)]
    _launch_emu(ctx, N.OP_RS, args, blocks or _emu_blocks(nbytes // W))
    ctx._stage = stage
    return outs


def emu_all_to_all(ctx: EmuContext, xs: list[torch.Tensor], blocks: int | None = None,
                   unroll: int = 0, push: bool = False) -> list[torch.Tensor]:
    W = ctx.world
    nbytes = xs[0].numel() * xs[0].element_size()
    stage = ctx.alloc(nbytes)
    outs = [torch.empty_like(x) for x in xs]
    sym = [s.data_ptr() for s in stage]
    args = [_fill_args(ctx.comms[r], sym, 0, xs[r].data_ptr(), outs[r].data_ptr(), nbytes,
                       copy_in=0 if push else 1, copy_out=1 if push else 0, unroll=unroll,
                       variant=1 if push else 0) for r in range(W)]
    _launch_emu(ctx, N.OP_A2A_FLAT, args, blocks or _emu_blocks(nbytes))
    ctx._stage = stage
    return outs


def emu_all_to_all_4d(ctx: EmuContext, xs: list[torch.Tensor], to_heads: bool,
                      blocks: int | None = None) -> list[torch.Tensor]:
    W = ctx.world
    x = xs[0]
    if to_heads:
        B, Sl, H, D = x.shape
        oshape = (B, Sl * W, H // W, D)
    else:
        B, S, Hl, D = x.shape
        Sl, H = S // W, Hl * W
        oshape = (B, Sl, H, D)
    nbytes = x.numel() * x.element_size()
    stage = ctx.alloc(nbytes)
    outs = [torch.empty(oshape, dtype=x.dtype, device=x.device) for _ in range(W)]
    sym = [s.data_ptr() for s in stage]
    geo = (B, Sl, H, D, 1 if to_heads else 0)
    args = [_fill_args(ctx.comms[r], sym, 0, xs[r].data_ptr(), outs[r].data_ptr(), nbytes,
                       copy_in=1, a2a=geo) for r in range(W)]
    _launch_emu(ctx, N.OP_A2A_4D, args, blocks or _emu_blocks(nbytes))
    ctx._stage = stage
    return outs


def emu_broadcast(ctx: EmuContext, xs: list[torch.Tensor], root: int = 0,
                  blocks: int | None = None) -> list[torch.Tensor]:
    W = ctx.world
    nbytes = xs[0].numel() * xs[0].element_size()
    stage = ctx.alloc(_pad16(nbytes))
    sym = [s.data_ptr() for s in stage]
    args = [_fill_args(ctx.comms[r], sym, 0, xs[r].data_ptr(), xs[r].data_ptr(), nbytes, copy_in=1,
                       root=root) for r in range(W)]
    _launch_emu(ctx, N.OP_BCAST, args, blocks or _emu_blocks(nbytes))
    ctx._stage = stage
    return xs


def emu_barrier(ctx: EmuContext, iters: int = 1):
    args = [_fill_args(ctx.comms[r], [], 0, 0, 0, 0) for r in range(ctx.world)]
    table = ctx.args_table(args)
    rc = ctx.lib.cb_barrier_launch(C.byref(args[0]), C.c_void_p(table.data_ptr()), ctx.world,
                                   iters, 0, N.stream_ptr())
    if rc != 0:
        raise CommError(f"emulated barrier launch failed: {N.last_error()}")
    ctx._keepalive = table
