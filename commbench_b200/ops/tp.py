"""Tensor-parallel fused GEMM + collective ops (one kernel each):

* :class:`AgGemm`  - all-gather(A rows) -> GEMM       (column-parallel linear)
* :class:`GemmRs`  - GEMM -> reduce-scatter(rows)      (row-parallel linear)
* :class:`GemmAr`  - GEMM -> all-reduce                (row-parallel linear, decode shapes)

Each object owns its symmetric staging buffers and flags (allocated once,
collectively), so a call is a single launch with no host synchronisation.
Weights follow the ``nn.Linear`` layout ``[out_features, in_features]``.

Reference counterparts: AllGatherMatmul / matmul_reduce_scatter / GEMM+AR of
datasets/example051_thunderkitten_ag_gemm_easy/nv/empty_thunderkitten_ag_gemm.cu:479-511,
datasets/example054_thunderkitten_gemm_rs_easy/nv/empty_thunderkitten_gemm_rs.cu:450-487,
datasets/example053_thunderkitten_gemm_ar_easy/nv/empty_thunderkitten_gemm_ar.cu:491-536.

Every class also accepts an :class:`~commbench_b200.runtime.context.EmuContext`; tensors are
then lists (one per virtual rank) and the call is one cooperative launch on one GPU.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N
from ..config import get_config
from ..runtime.context import CommContext, CommError, EmuContext
from ..utils.tracing import traced

_P8 = C.c_void_p * N.MAX_RANKS


class _AgDesc(C.Structure):
    _fields_ = [
        ("rank", C.c_int), ("world", C.c_int), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("fp8", C.c_int), ("alpha", C.c_float), ("bn", C.c_int), ("num_comm_ctas", C.c_int),
        ("parts", C.c_int), ("ctas_per_rank", C.c_int),
        ("a_local", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p),
        ("a_full_peer", _P8 * 2), ("a_full_mc", C.c_void_p * 2),
        ("flags_peer", _P8), ("flags_mc", C.c_void_p),
        ("seq", C.c_void_p), ("status", C.c_void_p), ("timeout_ns", C.c_ulonglong),
        ("a_sf_local", C.c_void_p), ("a_sf_full_peer", _P8 * 2), ("b_sf", C.c_void_p),
        ("src_ready", C.c_void_p), ("src_ready_target", C.c_uint), ("src_ready_rows", C.c_int),
    ]


class _RsDesc(C.Structure):
    _fields_ = [
        ("rank", C.c_int), ("world", C.c_int), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("fp8", C.c_int), ("alpha", C.c_float), ("bn", C.c_int), ("ctas_per_rank", C.c_int),
        ("a", C.c_void_p), ("b", C.c_void_p), ("out", C.c_void_p),
        ("stage_peer", _P8 * 2), ("flags_peer", _P8),
        ("seq", C.c_void_p), ("status", C.c_void_p), ("timeout_ns", C.c_ulonglong),
        ("a_sf", C.c_void_p), ("b_sf", C.c_void_p),
    ]


class _ArDesc(C.Structure):
    _fields_ = [
        ("rank", C.c_int), ("world", C.c_int), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("fp8", C.c_int), ("alpha", C.c_float), ("bn", C.c_int), ("oneshot", C.c_int),
        ("slots", C.c_int), ("ctas_per_rank", C.c_int),
        ("a", C.c_void_p), ("b", C.c_void_p), ("out", C.c_void_p),
        ("stage_peer", _P8 * 2), ("result_peer", _P8 * 2), ("result_mc", C.c_void_p * 2),
        ("flags_peer", _P8), ("seq", C.c_void_p), ("status", C.c_void_p),
        ("timeout_ns", C.c_ulonglong), ("trace", C.c_void_p),
        ("poll_ns", C.c_int),
    ]


import contextlib

_nullctx = contextlib.nullcontext


def _esz(dtype) -> int:
    return 1 if dtype == torch.float8_e4m3fn else 2


class _Sym:
    """A symmetric buffer seen uniformly for real and emulated contexts."""

    def __init__(self, ctx, nbytes: int, zero: bool = False):
        self.nbytes = nbytes
        if isinstance(ctx, EmuContext):
            self.tensors = ctx.alloc(nbytes)
            self.ptrs = [t.data_ptr() for t in self.tensors]
            self.mc = 0
        else:
            blk = ctx.alloc(nbytes)
            self.tensors = [blk.local]
            self.ptrs = blk.peer_ptrs
            self.mc = blk.mc_ptr
            if zero:
                blk.local.zero_()

    def local(self, ctx, r: int = 0) -> torch.Tensor:
        return self.tensors[r] if isinstance(ctx, EmuContext) else self.tensors[0]


def _fill_p8(arr, ptrs):
    for r in range(N.MAX_RANKS):
        arr[r] = ptrs[r] if r < len(ptrs) else 0


def _sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


class _FusedBase:
    def __init__(self, ctx):
        self.ctx = ctx
        self.lib = ctx.lib
        self.emu = isinstance(ctx, EmuContext)
        self.world = ctx.world
        self.nseq = ctx.world if self.emu else 1
        # {call counter, done CTAs} per (virtual) rank, local memory
        self.seq = [torch.zeros(4, dtype=torch.int32, device=ctx.device) for _ in range(self.nseq)]
        self.calls = 0
        self._table = None

    def _status_ptr(self, r: int) -> int:
        return self.ctx.comms[r].status if self.emu else self.ctx.comm.status

    def _ctas(self) -> int:
        sms = _sm_count(self.ctx.device)
        n = sms // self.world if self.emu else sms
        return n - n % 2      # CTA-pair tiles run as clusters of two

    def _pick_bn(self, M: int, Nn: int) -> int:
        """512 = a CTA pair (`tcgen05.mma.cta_group::2`) per 256 x 256 tile, the fastest form,
        whenever every rank owns whole 256-row blocks and there is at least one wave of such
        tiles; otherwise one CTA per 128 x 256 tile."""
        if M % (self.world * 256) == 0 and (M // 256) * ((Nn + 255) // 256) * 2 >= self._ctas():
            return 512
        return 256

    def _sync_init(self):
        torch.cuda.synchronize(self.ctx.device)
        if not self.emu:
            self.ctx.host_barrier()

    def _emu_table(self, nbytes: int):
        if self._table is None or self._table.numel() < nbytes:
            self._table = torch.empty(nbytes, dtype=torch.uint8, device=self.ctx.device)
        return C.c_void_p(self._table.data_ptr())


class AgGemm(_FusedBase):
    """``C[M, N_local] = all_gather_rows(A_local)[M, K] @ B[N_local, K].T`` in one kernel."""

    def __init__(self, ctx, max_m: int, k: int, dtype=torch.bfloat16):
        super().__init__(ctx)
        self.max_m, self.k, self.dtype = max_m, k, dtype
        nbytes = max_m * k * _esz(dtype)
        self.a_full = [_Sym(ctx, nbytes), _Sym(ctx, nbytes)]
        self.flags = _Sym(ctx, 2 * 1024 * 4, zero=True)
        # fp8 with hardware block scales: the gathered rows' packed scale words, per parity
        cfg = get_config()
        self.lib.cb_ag_gemm_set_row_poll_ns(C.c_uint(cfg.ag_gemm_row_poll_ns))
        self.lib.cb_ag_gemm_set_gate_poll_ns(C.c_uint(cfg.ag_gemm_gate_poll_ns))
        self.sf_full = None
        if dtype == torch.float8_e4m3fn and k % 128 == 0:
            sf_bytes = ((k // 128 + 3) // 4) * max_m * 4
            self.sf_full = [_Sym(ctx, sf_bytes), _Sym(ctx, sf_bytes)]
        self._sync_init()

    def _desc(self, r, a_local, b, c, M, Nn, K, alpha, bn, comm_ctas, parts, use_mc=True,
              a_sf=None, b_sf=None) -> _AgDesc:
        d = _AgDesc()
        d.rank, d.world, d.M, d.N, d.K = r, self.world, M, Nn, K
        d.fp8 = int(self.dtype == torch.float8_e4m3fn)
        d.alpha, d.bn = alpha, bn
        d.num_comm_ctas, d.parts, d.ctas_per_rank = comm_ctas, parts, self._ctas()
        d.a_local, d.b, d.c = a_local.data_ptr(), b.data_ptr(), c.data_ptr()
        for par in range(2):
            _fill_p8(d.a_full_peer[par], self.a_full[par].ptrs)
            d.a_full_mc[par] = self.a_full[par].mc if use_mc else 0
        _fill_p8(d.flags_peer, self.flags.ptrs)
        d.flags_mc = self.flags.mc if use_mc else 0
        d.seq = self.seq[r if self.emu else 0].data_ptr()
        d.status = self._status_ptr(r)
        d.timeout_ns = self.ctx.timeout_ns
        if a_sf is not None:
            d.a_sf_local, d.b_sf = a_sf.data_ptr(), b_sf.data_ptr()
            for par in range(2):
                _fill_p8(d.a_sf_full_peer[par], self.sf_full[par].ptrs)
        return d

    def pick_tiles(self, M: int, Nn: int) -> int:
        """Tile form of an all-gather GEMM on real ranks.  CTA pairs (256 x 256) are the faster
        main loop, but their row block - the unit a tile waits for - is 256 rows.  When a
        rank's OWN rows give less than one wave of pair tiles, the first remote row blocks
        are needed almost at once and the finer 128-row blocks of one-CTA tiles overlap
        better: measured on 8 GPUs (8192 x 3584 x 8192 per rank) 0.409 ms against 0.452 ms;
        on 4 GPUs (8192 x 7168) pairs win, 0.68-0.73 against 0.86 ms."""
        bn = self._pick_bn(M, Nn)
        if bn == 512 and self.world > 1 and not self.emu:
            local_tiles = (M // self.world // 256) * ((Nn + 255) // 256)
            if local_tiles < self._ctas() // 2:
                return 256
        return bn

    @staticmethod
    def pick_comm_ctas(M: int, Nn: int, bn: int, ctas: int, at_least: int, cap: int = 24) -> int:
        """Communication CTAs for a launch of ``ctas`` CTAs: the LARGEST even count up to
        ``cap`` that does not add a wave of tiles to the compute CTAs (8192 x 14336 in pair
        tiles = 1792 tiles: 72 pairs need 25 waves, 70 need 26, so 4 are taken; 8192 x 7168:
        10).  Multicast pushes do not get faster with more CTAs - on 8 GPUs 4 communication
        CTAs gave 0.409-0.452 ms and 20 gave 0.48-0.51 - so the caller caps the count at 4
        from 8 ranks up."""
        at_least = min(at_least, cap)
        pair = 2 if bn in (512, 192) else 1
        tile_m = 128 * pair
        tile_n = {512: 256, 192: 192}.get(bn, bn)
        tiles = ((M + tile_m - 1) // tile_m) * ((Nn + tile_n - 1) // tile_n)

        def waves(c):
            workers = (ctas - c) // pair
            return -(-tiles // workers) if workers > 0 else 1 << 30
        best, best_w = None, None
        for c in range(2, cap + 2, 2):
            w = waves(c)
            if best is None or w < best_w or (w == best_w and c >= best):
                if w < (best_w or 1 << 30) or c <= cap:
                    best, best_w = c, w
        # never below the floor unless that saves a whole wave
        if best < at_least and waves(at_least) == best_w:
            best = at_least
        return best

    @traced("cb200.ag_gemm")
    def __call__(self, a_local, b, out=None, alpha: float = 1.0, bn: int | None = None,
                 comm_ctas: int | None = None, parts: int | None = None, use_mc: bool = True,
                 stream=None, a_sf=None, b_sf=None, src_ready=None):
        """``a_sf`` / ``b_sf``: packed power-of-two block scales of fp8 operands
        (``ops.gemm.quantize_blockscaled_pow2``; ``a_sf`` of the LOCAL rows): the tensor cores
        apply them (``bn`` is then 192, CTA pairs on 256 x 192 tiles) and the scale words of a
        row block travel to the peers with its rows.

        ``src_ready = (words, target, rows_per_word)``: the local rows may still be arriving
        (a host-to-device copy in flight on another stream) when the kernel starts; int32 word
        ``r // rows_per_word`` of the CUDA tensor ``words`` reaches ``target`` once local row r
        has landed (:func:`stream_write_u32` after each chunk of the copy).  The kernel pushes
        and multiplies each row block as soon as its rows are there (real ranks only)."""
        cfg = get_config()
        auto_comm = comm_ctas is None
        if comm_ctas is None:
            comm_ctas = cfg.ag_gemm_comm_ctas if self.world > 1 else 0
        if self.emu:
            comm_ctas = min(comm_ctas, 4) if self.world > 1 else 0
        comm_ctas += comm_ctas % 2
        if parts is None and not (auto_comm and not self.emu and self.world > 1):
            parts = max(comm_ctas, 1)   # every comm CTA works on the same row block
        if self.emu:
            a0, b0 = a_local[0], b[0]
        else:
            a0, b0 = a_local, b
        Ml, K = a0.shape
        Nn = b0.shape[0]
        M = Ml * self.world
        if M > self.max_m or K != self.k:
            raise CommError(f"AgGemm built for M<={self.max_m}, K={self.k}; got M={M}, K={K}")
        if a_sf is not None:
            if self.sf_full is None or b_sf is None or M % (self.world * 256):
                raise CommError("block-scaled AgGemm: build it with dtype float8_e4m3fn, pass both "
                                "scale tensors, and shard whole 256-row blocks")
            bn = 192
        elif bn is None:
            bn = self.pick_tiles(M, Nn)
        if auto_comm and not self.emu and self.world > 1:
            comm_ctas = self.pick_comm_ctas(M, Nn, bn, self._ctas(), comm_ctas,
                                            cap=4 if self.world >= 8 else 24)
            if parts is None or parts < 1:
                parts = comm_ctas
        if self.emu:
            outs = out or [torch.empty((M, Nn), dtype=torch.bfloat16, device=a0.device)
                           for _ in range(self.world)]
            descs = (_AgDesc * self.world)(*[
                self._desc(r, a_local[r], b[r], outs[r], M, Nn, K, alpha, bn, comm_ctas, parts,
                           True, a_sf[r] if a_sf is not None else None,
                           b_sf[r] if b_sf is not None else None)
                for r in range(self.world)])
            table = self._emu_table(self.lib.cb_sizeof_ag_gemm_params() * self.world)
            rc = self.lib.cb_ag_gemm(descs, self.world, table, N.stream_ptr(stream))
            result = outs
        else:
            if out is None:
                out = torch.empty((M, Nn), dtype=torch.bfloat16, device=a0.device)
            descs = (_AgDesc * 1)(self._desc(self.ctx.rank, a_local, b, out, M, Nn, K, alpha, bn,
                                             comm_ctas, parts, use_mc, a_sf, b_sf))
            if src_ready is not None:
                words, target, rows_per_word = src_ready
                if words.dtype != torch.int32 or not words.is_cuda or \
                        words.numel() * rows_per_word < Ml:
                    raise CommError("src_ready: int32 CUDA words covering every local row")
                descs[0].src_ready = words.data_ptr()
                descs[0].src_ready_target = int(target) & 0xffffffff
                descs[0].src_ready_rows = int(rows_per_word)
            rc = self.lib.cb_ag_gemm(descs, 1, None, N.stream_ptr(stream))
            result = out
        if rc != 0:
            raise CommError(f"ag_gemm failed: {N.last_error()}")
        self.calls += 1
        return result


def stream_write_u32(word: torch.Tensor, value: int, stream=None) -> None:
    """Writes ``value`` into the one-element int32 CUDA tensor ``word`` when ``stream`` (default:
    the current stream) reaches this point - a stream memory operation, no kernel, so it
    completes even while a persistent kernel occupies every SM."""
    lib = N.load()
    if lib.cb_stream_write_u32(N.stream_ptr(stream), C.c_void_p(word.data_ptr()),
                               C.c_uint(int(value) & 0xffffffff)) != 0:
        raise CommError(f"stream_write_u32 failed: {N.last_error()}")


class GemmRs(_FusedBase):
    """``out[M/W, N] = reduce_scatter_rows(A[M, K_local] @ B[N, K_local].T)`` in one kernel."""

    def __init__(self, ctx, max_m: int, max_n: int):
        super().__init__(ctx)
        self.max_m, self.max_n = max_m, max_n
        self.lib.cb_gemm_rs_set_poll_ns(C.c_uint(get_config().gemm_rs_poll_ns))
        nbytes = max_m * max_n * 2  # W sources x M/W rows x N bf16
        self.stage = [_Sym(ctx, nbytes), _Sym(ctx, nbytes)]
        self.flags = _Sym(ctx, 2 * 8192 * 4, zero=True)
        self._sync_init()

    def _desc(self, r, a, b, out, M, Nn, K, alpha, bn, fp8, a_sf=None, b_sf=None) -> _RsDesc:
        d = _RsDesc()
        d.rank, d.world, d.M, d.N, d.K = r, self.world, M, Nn, K
        d.fp8, d.alpha, d.bn, d.ctas_per_rank = int(fp8), alpha, bn, self._ctas()
        d.a, d.b, d.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
        for par in range(2):
            _fill_p8(d.stage_peer[par], self.stage[par].ptrs)
        _fill_p8(d.flags_peer, self.flags.ptrs)
        d.seq = self.seq[r if self.emu else 0].data_ptr()
        d.status = self._status_ptr(r)
        d.timeout_ns = self.ctx.timeout_ns
        if a_sf is not None:
            d.a_sf, d.b_sf = a_sf.data_ptr(), b_sf.data_ptr()
        return d

    @traced("cb200.gemm_rs")
    def __call__(self, a, b, out=None, alpha: float = 1.0, bn: int | None = None, stream=None,
                 a_sf=None, b_sf=None):
        """``a_sf`` / ``b_sf``: packed power-of-two block scales of fp8 operands
        (``ops.gemm.quantize_blockscaled_pow2``), applied by the tensor cores."""
        a0, b0 = (a[0], b[0]) if self.emu else (a, b)
        M, K = a0.shape
        Nn = b0.shape[0]
        if M > self.max_m or Nn > self.max_n:
            raise CommError(f"GemmRs built for M<={self.max_m}, N<={self.max_n}")
        if a_sf is not None:
            if b_sf is None or M % (self.world * 256):
                raise CommError("block-scaled GemmRs: pass both scale tensors and shard whole "
                                "256-row blocks")
            bn = 192
        elif bn is None:
            bn = self._pick_bn(M, Nn)
        fp8 = a0.dtype == torch.float8_e4m3fn
        Ml = M // self.world
        if self.emu:
            outs = out or [torch.empty((Ml, Nn), dtype=torch.bfloat16, device=a0.device)
                           for _ in range(self.world)]
            descs = (_RsDesc * self.world)(*[
                self._desc(r, a[r], b[r], outs[r], M, Nn, K, alpha, bn, fp8,
                           a_sf[r] if a_sf is not None else None,
                           b_sf[r] if b_sf is not None else None)
                for r in range(self.world)])
            table = self._emu_table(self.lib.cb_sizeof_gemm_rs_params() * self.world)
            rc = self.lib.cb_gemm_rs(descs, self.world, table, N.stream_ptr(stream))
            result = outs
        else:
            if out is None:
                out = torch.empty((Ml, Nn), dtype=torch.bfloat16, device=a0.device)
            descs = (_RsDesc * 1)(self._desc(self.ctx.rank, a, b, out, M, Nn, K, alpha, bn, fp8,
                                             a_sf, b_sf))
            rc = self.lib.cb_gemm_rs(descs, 1, None, N.stream_ptr(stream))
            result = out
        if rc != 0:
            raise CommError(f"gemm_rs failed: {N.last_error()}")
        self.calls += 1
        return result


class GemmAr(_FusedBase):
    """``out[M, N] = all_reduce(A[M, K_local] @ B[N, K_local].T)``.

    ``mode="fused"``: one kernel (two-shot or one-shot epilogue).  ``mode="split"``: this
    package's GEMM into a symmetric buffer followed by its in-place all-reduce - two launches, no
    library kernel.  ``mode=None`` picks: measured on B200, the fused kernel wins on 8 ranks
    (1.1-1.5x cuBLAS + NCCL at M = 16 ... 1024) but on 2 and 4 ranks its three NVLink hops are
    not hidden behind so little math (0.55-0.98x), while the two tuned launches are ahead of
    the library pair there; so up to ``gemm_ar_split_max_world`` ranks "auto" means split."""

    def __init__(self, ctx, max_m: int, max_n: int):
        super().__init__(ctx)
        self.max_m, self.max_n = max_m, max_n
        # Worst case: one-shot, 64-wide tiles: every tile has a slot for every source.
        self.max_tiles = ((max_m + 127) // 128) * ((max_n + 63) // 64)
        self.stage_bytes = self.world * self.max_tiles * 128 * 64 * 2
        self.stage = [_Sym(ctx, self.stage_bytes), _Sym(ctx, self.stage_bytes)]
        self.result = [_Sym(ctx, max_m * max_n * 2), _Sym(ctx, max_m * max_n * 2)]
        self.flags = _Sym(ctx, self.lib.cb_gemm_ar_flag_words() * 4, zero=True)
        self.trace = None
        self.poll_ns = get_config().fused_poll_ns
        self._split_calls = 0
        self._sync_init()

    def _split(self, a, b, out, alpha, stream):
        """GEMM into one of the two symmetric result buffers, all-reduce in place."""
        from . import collectives as coll
        from .gemm import gemm

        M, Nn = a.shape[0], b.shape[0]
        buf = self.result[self._split_calls & 1].tensors[0]
        view = buf[: M * Nn * 2].view(torch.bfloat16).view(M, Nn)
        self._split_calls += 1
        gemm(a, b, out=view, alpha=alpha, stream=stream)
        coll.all_reduce(self.ctx, view, stream=stream)
        if out is None:
            return view
        with torch.cuda.stream(stream) if stream is not None else _nullctx():
            out.copy_(view)
        return out

    def _desc(self, r, a, b, out, M, Nn, K, alpha, bn, fp8, oneshot) -> _ArDesc:
        d = _ArDesc()
        d.rank, d.world, d.M, d.N, d.K = r, self.world, M, Nn, K
        d.fp8, d.alpha, d.bn, d.oneshot = int(fp8), alpha, bn, int(oneshot)
        d.slots = self.stage_bytes // (self.world * 128 * bn * 2)
        d.ctas_per_rank = self._ctas()
        d.a, d.b = a.data_ptr(), b.data_ptr()
        d.out = out.data_ptr() if out is not None else 0
        for par in range(2):
            _fill_p8(d.stage_peer[par], self.stage[par].ptrs)
            _fill_p8(d.result_peer[par], self.result[par].ptrs)
            d.result_mc[par] = self.result[par].mc
        _fill_p8(d.flags_peer, self.flags.ptrs)
        d.seq = self.seq[r if self.emu else 0].data_ptr()
        d.status = self._status_ptr(r)
        d.timeout_ns = self.ctx.timeout_ns
        d.trace = self.trace.data_ptr() if self.trace is not None else 0
        d.poll_ns = self.poll_ns
        return d

    def enable_trace(self) -> torch.Tensor:
        """Per-CTA phase time stamps (``%globaltimer`` ns) of the next calls: [ctas, 8] with
        columns start, GEMM phase done, own reductions done, all tiles done, exit."""
        dev = self.ctx.device
        self.trace = torch.zeros(_sm_count(dev), 8, dtype=torch.int64, device=dev)
        return self.trace

    @staticmethod
    def pick_bn(M: int, Nn: int, sms: int) -> int:
        mb = (M + 127) // 128
        for bn in (256, 128):
            if mb * ((Nn + bn - 1) // bn) >= 2 * sms:
                return bn
        return 64

    @traced("cb200.gemm_ar")
    def __call__(self, a, b, out=None, alpha: float = 1.0, bn: int | None = None,
                 oneshot: bool | None = None, stream=None, mode: str | None = None):
        a0, b0 = (a[0], b[0]) if self.emu else (a, b)
        M, K = a0.shape
        Nn = b0.shape[0]
        if M > self.max_m or Nn > self.max_n:
            raise CommError(f"GemmAr built for M<={self.max_m}, N<={self.max_n}")
        fp8 = a0.dtype == torch.float8_e4m3fn
        cfg = get_config()
        if mode is None:
            mode = "split" if (not self.emu and oneshot is None and bn is None and
                               1 < self.world <= cfg.gemm_ar_split_max_world) else "fused"
        if mode == "split":
            if self.emu:
                raise CommError("GemmAr mode='split' runs on real ranks")
            return self._split(a, b, out, alpha, stream)
        if mode != "fused":
            raise CommError(f"unknown GemmAr mode {mode!r}")
        if oneshot is None:
            # One-shot sends every partial tile to every rank (W times the traffic) and has one
            # polling CTA per tile.  Measured on 8 GPUs it loses at every M (116 us against 39 us
            # at M=16); with 2 ranks it is at best a few microseconds ahead and sometimes far
            # behind, so it is opt-in (gemm_ar_oneshot_max_m > 0).
            oneshot = M <= cfg.gemm_ar_oneshot_max_m
        if bn is None:
            bn = self.pick_bn(M, Nn, self._ctas())
        par = self.calls & 1            # the kernel derives the same parity from its call counter

        def sym_view(r):
            t = self.result[par].tensors[r if self.emu else 0]
            return t[: M * Nn * 2].view(torch.bfloat16).view(M, Nn)

        if self.emu:
            outs = out
            if oneshot and outs is None:
                outs = [torch.empty((M, Nn), dtype=torch.bfloat16, device=a0.device)
                        for _ in range(self.world)]
            descs = (_ArDesc * self.world)(*[
                self._desc(r, a[r], b[r], outs[r] if oneshot else None, M, Nn, K, alpha, bn, fp8,
                           oneshot)
                for r in range(self.world)])
            table = self._emu_table(self.lib.cb_sizeof_gemm_ar_params() * self.world)
            rc = self.lib.cb_gemm_ar(descs, self.world, table, N.stream_ptr(stream))
        else:
            if oneshot and out is None:
                out = torch.empty((M, Nn), dtype=torch.bfloat16, device=a0.device)
            descs = (_ArDesc * 1)(self._desc(self.ctx.rank, a, b, out if oneshot else None, M, Nn,
                                             K, alpha, bn, fp8, oneshot))
            rc = self.lib.cb_gemm_ar(descs, 1, None, N.stream_ptr(stream))
        if rc != 0:
            raise CommError(f"gemm_ar failed: {N.last_error()}")
        self.calls += 1
        if oneshot:
            return outs if self.emu else out
        # Two-shot: the reduced tensor sits in this call's symmetric result buffer.  Without
        # `out` a view of it is returned; it stays valid until the call after the next one.
        if self.emu:
            views = [sym_view(r) for r in range(self.world)]
            if out is None:
                return views
            for o, v in zip(out, views):
                o.copy_(v)
            return out
        if out is None:
            return sym_view(0)
        with torch.cuda.stream(stream) if stream is not None else _nullctx():
            out.copy_(sym_view(0))
        return out
