"""Python face of the native message transport (``csrc/util/transport.h``): endpoints with
verbs semantics on a loopback backend (always there) or libibverbs (when built with it).

It covers the API surface the reference's RDMA examples exercise against raw verbs - RC / UC /
UD queue pairs, RDMA write / read, send / recv, write-with-immediate (also zero-byte), inline
and scatter-gather sends, shared receive queues, atomics, memory windows, asynchronous CQ
errors, the device clock, device info and a registered-memory pool
(datasets/example002_rdma_loopback ... example029_ibv_query_qp_data_in_order; the pool is
datasets/example015_memory_pool_with_registered_region/empty_memory_pool.cpp:30-65) - plus the
TCP exchange of queue-pair addresses two processes use to find each other
(datasets/example006_rdma_read_write_rc/empty_rdma_read_write_rc.cpp:67,150-205).

Buffers are anything exposing a writable address: ``bytearray`` / ``numpy`` arrays / CPU or CUDA
``torch`` tensors.
"""
from __future__ import annotations

import ctypes as C
import json
import socket
import struct
from dataclasses import dataclass

from .. import _native as N

LOOPBACK, VERBS = 0, 1
RC, UC, UD = 0, 1, 2
SEND, SEND_IMM, WRITE, WRITE_IMM, READ, ATOMIC_CAS, ATOMIC_FADD, BIND_MW, LOCAL_INV = range(9)
RECV, RECV_IMM = 64, 65
LOCAL_WRITE, REMOTE_WRITE, REMOTE_READ, REMOTE_ATOMIC, MW_BIND = 1, 2, 4, 8, 16
ALL_ACCESS = 31
SIGNALED, INLINE = 1, 2
OK, LOC_LEN_ERR, LOC_PROT_ERR, REM_ACCESS_ERR, REM_INV_REQ_ERR, RNR_RETRY_EXC, WR_FLUSH_ERR = range(7)
EVENT_NONE, EVENT_CQ_ERR, EVENT_QP_FATAL = 0, 1, 2
MAX_SGE, UD_HEADER, UD_MTU = 16, 40, 4096


class TransportError(RuntimeError):
    pass


class _Sge(C.Structure):
    _fields_ = [("addr", C.c_uint64), ("length", C.c_uint32), ("lkey", C.c_uint32)]


class Addr(C.Structure):
    """What a peer needs to reach a queue pair."""
    _fields_ = [("qpn", C.c_uint32), ("psn", C.c_uint32), ("qkey", C.c_uint32), ("lid", C.c_uint32),
                ("gid", C.c_uint8 * 16)]

    def pack(self) -> bytes:
        return bytes(self)

    @classmethod
    def unpack(cls, raw: bytes) -> "Addr":
        return cls.from_buffer_copy(raw)


class _SendWr(C.Structure):
    _fields_ = [("wr_id", C.c_uint64), ("opcode", C.c_int), ("flags", C.c_int), ("num_sge", C.c_int),
                ("sge", _Sge * MAX_SGE), ("imm", C.c_uint32), ("remote_addr", C.c_uint64),
                ("rkey", C.c_uint32), ("compare_add", C.c_uint64), ("swap", C.c_uint64),
                ("ud_dest", Addr), ("mw_id", C.c_uint32), ("bind_lkey", C.c_uint32),
                ("bind_addr", C.c_uint64), ("bind_length", C.c_uint64), ("bind_access", C.c_int)]


class _Completion(C.Structure):
    _fields_ = [("wr_id", C.c_uint64), ("status", C.c_int), ("opcode", C.c_int),
                ("byte_len", C.c_uint32), ("imm", C.c_uint32), ("src_qpn", C.c_uint32),
                ("qpn", C.c_uint32)]


@dataclass
class Completion:
    wr_id: int
    status: int
    opcode: int
    byte_len: int
    imm: int
    src_qpn: int
    qpn: int

    @property
    def ok(self) -> bool:
        return self.status == OK


def buffer_address(buf) -> tuple[int, int]:
    """(address, nbytes) of a bytearray, numpy array or torch tensor."""
    if hasattr(buf, "data_ptr"):
        return int(buf.data_ptr()), int(buf.numel() * buf.element_size())
    if hasattr(buf, "ctypes") and hasattr(buf, "nbytes"):
        return int(buf.ctypes.data), int(buf.nbytes)
    if isinstance(buf, bytearray):
        c = (C.c_char * len(buf)).from_buffer(buf)
        return C.addressof(c), len(buf)
    raise TransportError(f"cannot take the address of a {type(buf).__name__}")


@dataclass
class MemoryRegion:
    addr: int
    length: int
    lkey: int
    rkey: int
    keepalive: object = None

    def sge(self, offset: int = 0, length: int | None = None) -> tuple[int, int, int]:
        length = self.length - offset if length is None else length
        if offset < 0 or offset + length > self.length:
            raise TransportError("scatter-gather entry outside the region")
        return (self.addr + offset, length, self.lkey)


def _lib():
    lib = N.load()
    if not getattr(lib, "_tp_ready", False):
        lib.cb_tp_open.restype = C.c_uint64
        lib.cb_tp_open.argtypes = [C.c_int, C.c_char_p]
        lib.cb_tp_close.argtypes = [C.c_uint64]
        lib.cb_tp_close.restype = None
        u64, u32, i32 = C.c_uint64, C.c_uint32, C.c_int
        P = C.POINTER
        sigs = {
            "cb_tp_device_info_json": [u64, C.c_char_p, i32],
            "cb_tp_query_clock_ns": [u64, P(u64)],
            "cb_tp_reg_mr": [u64, C.c_void_p, u64, i32, P(u32), P(u32)],
            "cb_tp_dereg_mr": [u64, u32],
            "cb_tp_alloc_mw": [u64, P(u32)],
            "cb_tp_mw_rkey": [u64, u32, P(u32)],
            "cb_tp_dealloc_mw": [u64, u32],
            "cb_tp_create_cq": [u64, i32, P(u32)],
            "cb_tp_create_srq": [u64, i32, P(u32)],
            "cb_tp_create_qp": [u64, i32, u32, u32, u32, i32, i32, i32, P(Addr)],
            "cb_tp_query_max_inline": [u64, u32, P(i32)],
            "cb_tp_connect": [u64, u32, P(Addr)],
            "cb_tp_destroy_qp": [u64, u32],
            "cb_tp_post_send": [u64, u32, P(_SendWr)],
            "cb_tp_post_recv": [u64, u32, u64, P(_Sge), i32],
            "cb_tp_post_srq_recv": [u64, u32, u64, P(_Sge), i32],
            "cb_tp_poll_cq": [u64, u32, P(_Completion), i32, C.c_int64],
            "cb_tp_get_async_event": [u64, i32, P(i32), P(u32)],
            "cb_tp_ack_async_event": [u64],
            "cb_tp_backend_available": [i32],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = C.c_int
        lib._tp_ready = True
    return lib


def backend_available(backend: int) -> bool:
    return bool(_lib().cb_tp_backend_available(backend))


class Context:
    """One open adapter.  All loopback contexts of a process share one fabric."""

    def __init__(self, backend: int = LOOPBACK, device: str = ""):
        self.lib = _lib()
        self.h = self.lib.cb_tp_open(backend, device.encode())
        if not self.h:
            raise TransportError(N.last_error())
        self.backend = backend

    def _ck(self, rc: int, what: str):
        if rc != 0:
            raise TransportError(f"{what}: {N.last_error()}")

    def close(self):
        if self.h:
            self.lib.cb_tp_close(self.h)
            self.h = 0

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ------------------------------------------------------------------ device
    def device_info(self) -> dict:
        buf = C.create_string_buffer(4096)
        n = self.lib.cb_tp_device_info_json(self.h, buf, len(buf))
        if n < 0:
            raise TransportError("device_info failed")
        return json.loads(buf.value.decode())

    def clock_ns(self) -> int:
        v = C.c_uint64(0)
        self._ck(self.lib.cb_tp_query_clock_ns(self.h, C.byref(v)), "query_clock")
        return v.value

    # ------------------------------------------------------------------ memory
    def reg_mr(self, buf, access: int = ALL_ACCESS) -> MemoryRegion:
        addr, n = buffer_address(buf)
        lk, rk = C.c_uint32(0), C.c_uint32(0)
        self._ck(self.lib.cb_tp_reg_mr(self.h, C.c_void_p(addr), n, access, C.byref(lk), C.byref(rk)),
                 "reg_mr")
        return MemoryRegion(addr, n, lk.value, rk.value, buf)

    def dereg_mr(self, mr: MemoryRegion):
        self._ck(self.lib.cb_tp_dereg_mr(self.h, mr.lkey), "dereg_mr")

    def alloc_mw(self) -> int:
        v = C.c_uint32(0)
        self._ck(self.lib.cb_tp_alloc_mw(self.h, C.byref(v)), "alloc_mw")
        return v.value

    def mw_rkey(self, mw: int) -> int:
        v = C.c_uint32(0)
        self._ck(self.lib.cb_tp_mw_rkey(self.h, mw, C.byref(v)), "mw_rkey")
        return v.value

    def dealloc_mw(self, mw: int):
        self._ck(self.lib.cb_tp_dealloc_mw(self.h, mw), "dealloc_mw")

    # ------------------------------------------------------------------ queues
    def create_cq(self, depth: int = 256) -> int:
        v = C.c_uint32(0)
        self._ck(self.lib.cb_tp_create_cq(self.h, depth, C.byref(v)), "create_cq")
        return v.value

    def create_srq(self, depth: int = 256) -> int:
        v = C.c_uint32(0)
        self._ck(self.lib.cb_tp_create_srq(self.h, depth, C.byref(v)), "create_srq")
        return v.value

    def create_qp(self, qp_type: int = RC, send_cq: int | None = None, recv_cq: int | None = None,
                  srq: int = 0, max_send_wr: int = 128, max_recv_wr: int = 128,
                  max_inline: int = 0) -> "Endpoint":
        if send_cq is None:
            send_cq = self.create_cq()
        if recv_cq is None:
            recv_cq = send_cq
        a = Addr()
        self._ck(self.lib.cb_tp_create_qp(self.h, qp_type, send_cq, recv_cq, srq, max_send_wr,
                                          max_recv_wr, max_inline, C.byref(a)), "create_qp")
        return Endpoint(self, qp_type, a, send_cq, recv_cq, srq)

    def post_srq_recv(self, srq: int, wr_id: int, sges):
        arr = _sge_array(sges)
        self._ck(self.lib.cb_tp_post_srq_recv(self.h, srq, wr_id, arr, len(sges)), "post_srq_recv")

    def poll_cq(self, cq: int, max_entries: int = 16, timeout_us: int = 1_000_000) -> list[Completion]:
        out = (_Completion * max_entries)()
        n = self.lib.cb_tp_poll_cq(self.h, cq, out, max_entries, timeout_us)
        if n < 0:
            raise TransportError(f"poll_cq: {N.last_error()}")
        return [Completion(o.wr_id, o.status, o.opcode, o.byte_len, o.imm, o.src_qpn, o.qpn)
                for o in out[:n]]

    # ------------------------------------------------------------------ events
    def get_async_event(self, timeout_ms: int = 0) -> tuple[int, int] | None:
        ev, obj = C.c_int(0), C.c_uint32(0)
        got = self.lib.cb_tp_get_async_event(self.h, timeout_ms, C.byref(ev), C.byref(obj))
        if got < 0:
            raise TransportError(N.last_error())
        return (ev.value, obj.value) if got else None

    def ack_async_event(self):
        self._ck(self.lib.cb_tp_ack_async_event(self.h), "ack_async_event")


def _sge_array(sges):
    if len(sges) > MAX_SGE:
        raise TransportError(f"at most {MAX_SGE} scatter-gather entries")
    arr = (_Sge * max(len(sges), 1))()
    for i, (addr, length, lkey) in enumerate(sges):
        arr[i].addr, arr[i].length, arr[i].lkey = addr, length, lkey
    return arr


class Endpoint:
    """One queue pair."""

    def __init__(self, ctx: Context, qp_type: int, addr: Addr, send_cq: int, recv_cq: int, srq: int):
        self.ctx, self.type, self.addr = ctx, qp_type, addr
        self.send_cq, self.recv_cq, self.srq = send_cq, recv_cq, srq
        self.qpn = addr.qpn

    def connect(self, remote: Addr | None = None):
        ptr = C.byref(remote) if remote is not None else None
        self.ctx._ck(self.ctx.lib.cb_tp_connect(self.ctx.h, self.qpn, ptr), "connect")

    def destroy(self):
        self.ctx._ck(self.ctx.lib.cb_tp_destroy_qp(self.ctx.h, self.qpn), "destroy_qp")

    @property
    def max_inline(self) -> int:
        v = C.c_int(0)
        self.ctx._ck(self.ctx.lib.cb_tp_query_max_inline(self.ctx.h, self.qpn, C.byref(v)),
                     "query_max_inline")
        return v.value

    def post_recv(self, wr_id: int, sges):
        arr = _sge_array(sges)
        self.ctx._ck(self.ctx.lib.cb_tp_post_recv(self.ctx.h, self.qpn, wr_id, arr, len(sges)),
                     "post_recv")

    def post(self, opcode: int, sges=(), wr_id: int = 0, flags: int = SIGNALED, imm: int = 0,
             remote_addr: int = 0, rkey: int = 0, compare_add: int = 0, swap: int = 0,
             dest: Addr | None = None, mw: int = 0, bind: tuple | None = None):
        """Posts one send-side work request.  ``bind`` = (region, offset, length, access) for
        BIND_MW; ``mw`` is the window id (BIND_MW) or the remote key to kill (LOCAL_INV)."""
        wr = _SendWr()
        wr.wr_id, wr.opcode, wr.flags, wr.num_sge = wr_id, opcode, flags, len(sges)
        if len(sges) > MAX_SGE:
            raise TransportError(f"at most {MAX_SGE} scatter-gather entries")
        for i, (addr, length, lkey) in enumerate(sges):
            wr.sge[i].addr, wr.sge[i].length, wr.sge[i].lkey = addr, length, lkey
        wr.imm, wr.remote_addr, wr.rkey = imm, remote_addr, rkey
        wr.compare_add, wr.swap = compare_add, swap
        if dest is not None:
            wr.ud_dest = dest
        wr.mw_id = mw
        if bind is not None:
            region, off, length, access = bind
            wr.bind_lkey, wr.bind_addr, wr.bind_length, wr.bind_access = \
                region.lkey, region.addr + off, length, access
        self.ctx._ck(self.ctx.lib.cb_tp_post_send(self.ctx.h, self.qpn, C.byref(wr)), "post_send")

    def poll_send(self, **kw) -> list[Completion]:
        return self.ctx.poll_cq(self.send_cq, **kw)

    def poll_recv(self, **kw) -> list[Completion]:
        return self.ctx.poll_cq(self.recv_cq, **kw)


def connect_pair(a: Endpoint, b: Endpoint):
    """Both directions of a connected (RC / UC) pair."""
    a.connect(b.addr)
    b.connect(a.addr)


class MemoryPool:
    """One registration over a large buffer, handed out as slices from a stack allocator:
    ``alloc`` takes the next aligned slice, ``release`` returns the most recent ones."""

    def __init__(self, ctx: Context, buf, align: int = 256, access: int = ALL_ACCESS):
        self.ctx, self.align = ctx, align
        self.mr = ctx.reg_mr(buf, access)
        self.top = 0
        self.stack: list[int] = []

    def alloc(self, nbytes: int) -> tuple[int, int, int]:
        """(address, length, lkey) of a fresh slice."""
        absolute = (self.mr.addr + self.top + self.align - 1) // self.align * self.align
        start = absolute - self.mr.addr
        if start + nbytes > self.mr.length:
            raise TransportError("memory pool exhausted")
        self.stack.append(self.top)
        self.top = start + nbytes
        return self.mr.sge(start, nbytes)

    def release(self, count: int = 1):
        for _ in range(count):
            if not self.stack:
                raise TransportError("memory pool: nothing to release")
            self.top = self.stack.pop()

    @property
    def used(self) -> int:
        return self.top


# ----------------------------------------------------------------- out-of-band exchange
_META = struct.Struct("!32sQI")   # address blob, buffer address, remote key


def exchange_metadata(sock: socket.socket, addr: Addr, buf_addr: int = 0, rkey: int = 0):
    """Sends this side's (queue-pair address, buffer address, rkey) and returns the peer's, over
    a connected TCP socket - the hand-shake two processes do before they can use RDMA."""
    sock.sendall(_META.pack(addr.pack(), buf_addr, rkey))
    raw = b""
    while len(raw) < _META.size:
        chunk = sock.recv(_META.size - len(raw))
        if not chunk:
            raise TransportError("peer closed the metadata connection")
        raw += chunk
    blob, peer_buf, peer_rkey = _META.unpack(raw)
    return Addr.unpack(blob), peer_buf, peer_rkey


# ------------------------------------------------------- two-rank all-reduce over put + signal
class PutSignalAllReduce:
    """All-reduce between two ranks that are only connected by the transport (another node):
    put the local vector into the peer's receive window, bump the peer's signal counter with a
    remote atomic, flush, wait for the peer's signal, add.  The pattern of
    datasets/example092_nccl_device_api_internode_allreduce/
    empty_nccl_device_api_internode_allreduce.cu:47-87 (put with signal increment, wait on the
    signal, flush, local add), expressed on work requests instead of a vendor's device API.

    Each side: ``ar = PutSignalAllReduce(ctx, ep, numel)``; exchange ``ar.window()`` with the
    peer (``connect_window``); then per call ``ar.start(x)`` followed by ``ar.finish()``."""

    def __init__(self, ctx: Context, ep: Endpoint, numel: int):
        import numpy as np

        self.ctx, self.ep, self.numel = ctx, ep, numel
        self.send = np.zeros(numel, dtype=np.float32)
        self.recv = np.zeros(numel, dtype=np.float32)
        self.signal = np.zeros(1, dtype=np.uint64)
        self.scratch = np.zeros(1, dtype=np.uint64)
        self.m_send, self.m_recv = ctx.reg_mr(self.send), ctx.reg_mr(self.recv)
        self.m_sig, self.m_scr = ctx.reg_mr(self.signal), ctx.reg_mr(self.scratch)
        self.round = 0
        self.peer = None

    def window(self) -> tuple[int, int, int, int]:
        return (self.m_recv.addr, self.m_recv.rkey, self.m_sig.addr, self.m_sig.rkey)

    def connect_window(self, peer_window):
        self.peer = tuple(peer_window)

    def start(self, x):
        if self.peer is None:
            raise TransportError("connect_window() first")
        self.send[:] = x
        raddr, rkey, saddr, skey = self.peer
        self.round += 1
        self.ep.post(WRITE, [self.m_send.sge()], wr_id=2 * self.round, remote_addr=raddr, rkey=rkey)
        self.ep.post(ATOMIC_FADD, [self.m_scr.sge()], wr_id=2 * self.round + 1, remote_addr=saddr,
                     rkey=skey, compare_add=1)

    def finish(self, timeout_s: float = 10.0):
        import time as _time

        done = 0
        deadline = _time.monotonic() + timeout_s
        while done < 2:                                    # flush: both requests completed
            for c in self.ep.poll_send(timeout_us=100_000):
                if not c.ok:
                    raise TransportError(f"all-reduce put failed with status {c.status}")
                done += 1
            if _time.monotonic() > deadline:
                raise TransportError("all-reduce: flush timed out")
        while int(self.signal[0]) < self.round:            # the peer's put has landed
            if _time.monotonic() > deadline:
                raise TransportError("all-reduce: the peer's signal never arrived")
            _time.sleep(0)
        return self.send + self.recv
