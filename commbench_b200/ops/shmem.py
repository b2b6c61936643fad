"""One-sided operations on the symmetric heap (the NVSHMEM / MSCCL++ memory-channel style API):
``put_signal``, ``wait`` / ``wait_get``, ``atomic_fetch_inc``, ``tile_put`` / ``tile_consume``.

Addresses are plain device pointers; for a :class:`~commbench_b200.runtime.context.SymmBlock`
``blk.peer_ptrs[r]`` is rank r's copy.  The same functions work on two local buffers, which is
how the single-GPU tests exercise producer and consumer (as consecutive launches - the consumer
never has to wait for a later launch).

Reference counterparts: datasets/example033_nvshmem_put_and_signal, datasets/example038/039/040 and
090/096 (MSCCL++ put / get / signal), datasets/example032_nvshmem_atomic_fetch_inc,
datasets/example035_nvshmem_tiled_produce_consume, datasets/example034_nvshmem_broadcast (covered by
``ops.collectives.broadcast``).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N


class ShmemError(RuntimeError):
    pass


_scratch: dict = {}


def _done_word(device) -> torch.Tensor:
    key = str(device)
    if key not in _scratch:
        _scratch[key] = torch.zeros(4, dtype=torch.int32, device=device)
    return _scratch[key]


def put_signal(dst_ptr: int, src: torch.Tensor, signal_ptr: int = 0, value: int = 1,
               add: bool = False, blocks: int = 32, stream=None):
    """Copies ``src`` to ``dst_ptr`` (usually a peer's copy), then - after a release covering
    the whole copy - sets (or adds to) the signal word at ``signal_ptr``."""
    lib = N.load()
    nbytes = src.numel() * src.element_size()
    rc = lib.cb_shmem_put_signal(C.c_void_p(dst_ptr), N.ptr(src), C.c_longlong(nbytes),
                                 C.c_void_p(signal_ptr), C.c_uint(value), int(add),
                                 N.ptr(_done_word(src.device)), blocks, N.stream_ptr(stream))
    if rc != 0:
        raise ShmemError(N.last_error())


def wait_get(signal_ptr: int, value: int, dst: torch.Tensor | None = None, src_ptr: int = 0,
             timeout_s: float = 2.0, status: torch.Tensor | None = None, blocks: int = 32,
             stream=None):
    """Waits (bounded) until the signal word reaches ``value``; with ``dst`` also pulls
    ``dst.nbytes`` bytes from ``src_ptr``."""
    lib = N.load()
    nbytes = 0 if dst is None else dst.numel() * dst.element_size()
    rc = lib.cb_shmem_wait_get(N.ptr(dst), C.c_void_p(src_ptr), C.c_longlong(nbytes),
                               C.c_void_p(signal_ptr), C.c_uint(value),
                               C.c_ulonglong(int(timeout_s * 1e9)), N.ptr(status),
                               blocks if dst is not None else 1, N.stream_ptr(stream))
    if rc != 0:
        raise ShmemError(N.last_error())


def atomic_fetch_inc(counter_ptr: int, n: int, device=None):
    """``n`` fetch-and-increments on a 64-bit counter (possibly on another rank).  Returns
    (tickets [n] int64, cycles)."""
    lib = N.load()
    device = device or torch.device("cuda", torch.cuda.current_device())
    tickets = torch.empty(n, dtype=torch.int64, device=device)
    cyc = torch.zeros(1, dtype=torch.int64, device=device)
    rc = lib.cb_shmem_atomic_fetch_inc(C.c_void_p(counter_ptr), n, N.ptr(tickets), N.ptr(cyc),
                                       N.stream_ptr())
    if rc != 0:
        raise ShmemError(N.last_error())
    return tickets, cyc


def tile_put(dst_ptr: int, src: torch.Tensor, tile: int, flags_ptr: int, value: int = 1,
             stream=None):
    """``src`` is a square fp32 matrix; every ``tile x tile`` block is written into the matrix at
    ``dst_ptr`` and its flag raised, one CTA per tile."""
    lib = N.load()
    rc = lib.cb_shmem_tile_put(C.c_void_p(dst_ptr), N.ptr(src), src.shape[0], tile,
                               C.c_void_p(flags_ptr), C.c_uint(value), N.stream_ptr(stream))
    if rc != 0:
        raise ShmemError(N.last_error())


def tile_consume(m: torch.Tensor, tile: int, flags_ptr: int, value: int = 1, timeout_s: float = 2.0,
                 status: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """Per-tile sums of ``m`` taken as soon as each tile's flag is up."""
    lib = N.load()
    nt = (m.shape[0] // tile) ** 2
    partial = torch.zeros(nt, dtype=torch.float32, device=m.device)
    rc = lib.cb_shmem_tile_consume(N.ptr(m), m.shape[0], tile, C.c_void_p(flags_ptr),
                                   C.c_uint(value), N.ptr(partial),
                                   C.c_ulonglong(int(timeout_s * 1e9)), N.ptr(status),
                                   N.stream_ptr(stream))
    if rc != 0:
        raise ShmemError(N.last_error())
    return partial
