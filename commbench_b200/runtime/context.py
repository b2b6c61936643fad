"""Communicator context: symmetric heap, signal pad, status word.

One process drives one GPU.  :class:`CommContext` owns

* a *symmetric heap*: one VMM segment per rank, mapped by every peer and (when
  the fabric allows) bound to an NVSwitch multicast object, sub-allocated here so
  that the same allocation sequence yields the same offsets on every rank;
* the *signal pad* and the per-channel epoch counters the kernels synchronise on;
* a host-mapped *status word* that kernels set when a bounded wait runs out.

Capability parity with the reference: ParallelTensor + KittensBroker
(datasets/example048_thunderkitten_all_reduce_easy/nv/empty_thunderkitten_all_reduce.cu:161-243,
datasets/example060_thunderkitten_all_reduce_hard/nv/empty_thunderkitten_all_reduce.cu:112-146),
the cudaIpc hand-off (datasets/example012_gpu_ipc_comm_with_NVLink/nv/empty_gpu_ipc_comm.cu:110-180)
and NCCL symmetric windows (datasets/example043_nccl_device_api_intranode_allreduce/
empty_nccl_device_api_allreduce.cu:121-128).

:class:`EmuContext` keeps ``world`` *virtual* ranks on ONE GPU.  Its collectives
run as a single cooperative launch whose grid carries one slice per virtual
rank, so the cross-rank protocol (flags, barriers, peer pointers) is exercised
on a single device without ever running kernels that wait on each other as
separate launches.
"""
from __future__ import annotations

import ctypes as C
import os
import uuid
from dataclasses import dataclass

import torch

from .. import _native as N

_ALIGN = 1024  # TMA 128-byte swizzle wants 1024-byte aligned tiles
_CANARY = 0xA5


class CommError(RuntimeError):
    pass


class _RawCuda:
    """Minimal __cuda_array_interface__ carrier so torch can view raw device memory."""

    def __init__(self, ptr: int, nbytes: int, owner=None):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
            "strides": None,
        }
        self._owner = owner


def tensor_from_ptr(ptr: int, nbytes: int, device: torch.device, owner=None) -> torch.Tensor:
    return torch.as_tensor(_RawCuda(ptr, nbytes, owner), device=device)


@dataclass
class SymmBlock:
    """A block of the symmetric heap: the same offset on every rank."""

    offset: int
    nbytes: int
    local: torch.Tensor          # uint8 view of this rank's copy
    peer_ptrs: list[int]         # device addresses of every rank's copy (own included)
    mc_ptr: int                  # multicast alias or 0

    def view(self, dtype: torch.dtype, shape) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nb = n * torch.empty((), dtype=dtype).element_size()
        if nb > self.nbytes:
            raise CommError(f"view of {nb} bytes over a {self.nbytes}-byte block")
        return self.local[:nb].view(dtype).view(*shape)


class _ContextBase:
    rank: int
    world: int
    device: torch.device
    timeout_ns: int

    def _make_comm(self, rank, pads, mc_pad, epoch_ptr, status_dev_ptr) -> N.CbComm:
        c = N.CbComm()
        c.rank = rank
        c.world = self.world
        for r in range(N.MAX_RANKS):
            c.pad[r] = pads[r] if r < len(pads) else 0
        c.mc_pad = mc_pad
        c.epoch = epoch_ptr
        c.status = status_dev_ptr
        c.timeout_ns = self.timeout_ns
        # Debug stress (CB200_DEBUG_JITTER_NS): pseudo-random start delay per CTA in the
        # collective kernels; capped well below the wait budget.
        c.jitter_ns = min(int(os.environ.get("CB200_DEBUG_JITTER_NS", "0") or 0),
                          max(self.timeout_ns // 100, 0), 10_000_000)
        return c


class CommContext(_ContextBase):
    """Real multi-process context (one rank per process / GPU)."""

    def __init__(self, group=None, heap_bytes: int | None = None, use_multicast: bool | None = None,
                 timeout_s: float | None = None, device: torch.device | None = None):
        import torch.distributed as dist

        self.lib = N.load()
        if not torch.cuda.is_available():
            raise CommError("CommContext needs a CUDA device (use EmuContext tests or gloo paths on CPU)")
        self.dist = dist
        if dist.is_initialized():
            self.rank = dist.get_rank(group)
            self.world = dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        if self.world not in (1, 2, 4, 8):
            raise CommError(f"world size {self.world} not supported (1, 2, 4, 8)")
        self.group = group
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        torch.cuda.set_device(self.device)
        from ..config import get_config

        cfg = get_config()          # CB200_TIMEOUT_S, CB200_HEAP_BYTES, CB200_USE_NVLS
        self.timeout_ns = int((timeout_s if timeout_s is not None else cfg.timeout_s) * 1e9)
        self.heap_bytes = heap_bytes or int(cfg.heap_bytes)
        if use_multicast is None:   # CB200_NVLS=0 is the older spelling of CB200_USE_NVLS=0
            use_multicast = bool(cfg.use_nvls) and os.environ.get("CB200_NVLS", "1") != "0"
        self._ctrl = None
        if self.world > 1:
            # CPU control plane for object exchange (the NCCL group moves tensors only).
            self._ctrl = dist.new_group(backend="gloo") if dist.get_backend(group) != "gloo" else group
        self._broker = C.c_void_p(0)
        self._segments = []  # (handle, local_ptr, peer_ptrs, mc_ptr, nbytes, used)
        self._named: dict[str, SymmBlock] = {}
        self._canaries = [] if os.environ.get("CB200_DEBUG_CANARIES", "0") != "0" else None
        self.mode = "single"
        self.has_multicast = False
        self._closed = False
        if self.world > 1:
            self._start_broker()
        self._want_mc = bool(use_multicast) and self.world > 1 and \
            self.lib.cb_symm_multicast_supported(self.device.index or 0) == 1
        self._add_segment(self.heap_bytes)
        # Signal pad first, so its offset is identical everywhere.
        self.pad = self.alloc(N.PAD_WORDS * 4)
        self.pad.local.zero_()
        self.epoch = torch.zeros(N.PAD_CHANNELS, dtype=torch.int32, device=self.device)
        hp, dp = C.c_void_p(0), C.c_void_p(0)
        N.check(self.lib.cb_mapped_alloc(C.c_longlong(64), C.byref(hp), C.byref(dp)), "cb_mapped_alloc")
        self._status_host = (C.c_uint32 * 16).from_address(hp.value)
        self._status_host_ptr = hp
        self._status_dev = dp.value
        self.comm = self._make_comm(self.rank, self.pad.peer_ptrs, self.pad.mc_ptr,
                                    self.epoch.data_ptr(), self._status_dev)
        torch.cuda.synchronize(self.device)
        self.host_barrier()

    # ------------------------------------------------------------------ bootstrap
    def _bcast_obj(self, obj, src=0):
        box = [obj]
        self.dist.broadcast_object_list(box, src=src, group=self._ctrl)
        return box[0]

    def _allgather_obj(self, obj):
        out = [None] * self.world
        self.dist.all_gather_object(out, obj, group=self._ctrl)
        return out

    def _start_broker(self):
        name = self._bcast_obj(f"cb200-{os.getpid()}-{uuid.uuid4().hex[:12]}")
        self._job_name = name
        N.check(self.lib.cb_broker_create(name.encode(), self.rank, self.world, 30000,
                                          C.byref(self._broker)), "cb_broker_create")

    def host_barrier(self, timeout_ms: int = 60000):
        if self.world == 1:
            return
        rc = self.lib.cb_broker_barrier(self._broker, timeout_ms)
        if rc != 0:
            raise CommError(f"host barrier failed: {N.last_error()}")

    def _add_segment(self, want_bytes: int):
        lib = self.lib
        dev = self.device.index or 0
        if self.world == 1:
            nbytes = max(want_bytes, 1 << 21)
            buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            self._segments.append(dict(handle=None, tensor=buf, local=buf.data_ptr(),
                                       peers=[buf.data_ptr()], mc=0, nbytes=nbytes, used=0))
            self.mode = "single"
            return
        nbytes = lib.cb_symm_round_size(dev, C.c_longlong(want_bytes), self.world, int(self._want_mc))
        ok_vmm = nbytes > 0
        seg, local = C.c_void_p(0), C.c_void_p(0)
        fd = -1
        if ok_vmm:
            ok_vmm = lib.cb_symm_segment_create(dev, C.c_longlong(nbytes), C.byref(seg),
                                                C.byref(local)) == 0
        if ok_vmm:
            fd = lib.cb_symm_segment_export_fd(seg)
            ok_vmm = fd >= 0
        why = "" if ok_vmm else N.last_error()
        all_ok = all(self._allgather_obj(bool(ok_vmm)))
        if not all_ok:
            if seg.value:
                lib.cb_symm_segment_destroy(seg)
            self._add_segment_ipc(want_bytes, why)
            return
        fds = (C.c_int * N.MAX_RANKS)()
        N.check(lib.cb_broker_exchange_fds(self._broker, fd, fds, 60000), "cb_broker_exchange_fds")
        peers = [0] * self.world
        peers[self.rank] = local.value
        for r in range(self.world):
            if r != self.rank:
                p = C.c_void_p(0)
                N.check(lib.cb_symm_segment_import_peer(seg, r, fds[r], C.byref(p)),
                        f"import peer {r}")
                peers[r] = p.value
            os.close(fds[r])
        os.close(fd)
        self.host_barrier()
        mc_ptr = 0
        if self._want_mc:
            mc_ptr = self._bind_multicast(seg)
        self._segments.append(dict(handle=seg, tensor=None, local=local.value, peers=peers,
                                   mc=mc_ptr, nbytes=nbytes, used=0))
        self.mode = "vmm"
        self.has_multicast = mc_ptr != 0

    def _bind_multicast(self, seg) -> int:
        lib = self.lib
        ok = True
        fd = -1
        if self.rank == 0:
            fd = lib.cb_symm_mc_create(seg, self.world)
            ok = fd >= 0
        ok = bool(self._bcast_obj(ok))
        if not ok:
            self._want_mc = False
            return 0
        got = C.c_int(-1)
        N.check(lib.cb_broker_broadcast_fd(self._broker, 0, fd if self.rank == 0 else -1,
                                           C.byref(got), 60000), "cb_broker_broadcast_fd")
        if self.rank != 0:
            ok = lib.cb_symm_mc_import(seg, got.value) == 0
        os.close(got.value)
        if self.rank == 0:
            os.close(fd)
        if ok:
            ok = lib.cb_symm_mc_add_device(seg) == 0
        if not all(self._allgather_obj(bool(ok))):
            self._want_mc = False
            return 0
        self.host_barrier()
        mc = C.c_void_p(0)
        ok = lib.cb_symm_mc_bind(seg, C.byref(mc)) == 0
        if not all(self._allgather_obj(bool(ok))):
            self._want_mc = False
            return 0
        self.host_barrier()
        return mc.value or 0

    def _add_segment_ipc(self, want_bytes: int, why: str):
        """cudaIpc fallback: no fd passing, no multicast."""
        lib = self.lib
        nbytes = (want_bytes + (1 << 21) - 1) // (1 << 21) * (1 << 21)
        p = C.c_void_p(0)
        h = (C.c_ubyte * 64)()
        N.check(lib.cb_ipc_alloc(C.c_longlong(nbytes), C.byref(p), h), "cb_ipc_alloc")
        handles = self._allgather_obj(bytes(h))
        peers = [0] * self.world
        peers[self.rank] = p.value
        for r in range(self.world):
            if r != self.rank:
                q = C.c_void_p(0)
                hb = (C.c_ubyte * 64).from_buffer_copy(handles[r])
                N.check(lib.cb_ipc_open(hb, C.byref(q)), f"cb_ipc_open rank {r}")
                peers[r] = q.value
        self._segments.append(dict(handle=None, ipc=True, tensor=None, local=p.value, peers=peers,
                                   mc=0, nbytes=nbytes, used=0))
        self.mode = "ipc"
        self._want_mc = False
        self.vmm_failure = why

    # ------------------------------------------------------------------ allocator
    def alloc(self, nbytes: int) -> SymmBlock:
        """Collective: every rank calls it with the same size in the same order."""
        nbytes = max(int(nbytes), 16)
        # Debug build of the heap: one guard page of a known pattern on either side of every
        # block, verified by check_canaries() - an out-of-bounds peer store shows up there.
        guard = _ALIGN if self._canaries is not None else 0
        need = (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN + 2 * guard
        seg = self._segments[-1]
        if seg["used"] + need > seg["nbytes"]:
            self._add_segment(max(need, self.heap_bytes))
            seg = self._segments[-1]
        off = seg["used"] + guard
        seg["used"] += need
        if seg["tensor"] is not None:
            local = seg["tensor"][off:off + nbytes]
        else:
            local = tensor_from_ptr(seg["local"] + off, nbytes, self.device, owner=self)
        if guard:
            base = seg["local"] if seg["tensor"] is None else seg["tensor"].data_ptr()
            for g_off in (off - guard, off + need - 2 * guard):
                g = tensor_from_ptr(base + g_off, guard, self.device, owner=self)
                g.fill_(_CANARY)
                self._canaries.append((g, off, nbytes))
        return SymmBlock(offset=off, nbytes=nbytes, local=local,
                         peer_ptrs=[p + off for p in seg["peers"]],
                         mc_ptr=(seg["mc"] + off) if seg["mc"] else 0)

    def check_canaries(self):
        """Debug heaps only (``CB200_DEBUG_CANARIES=1``): raises if any guard page around a
        symmetric block was written to."""
        if not self._canaries:
            return
        torch.cuda.synchronize(self.device) if self.device.type == "cuda" else None
        for g, off, nbytes in self._canaries:
            if not bool((g == _CANARY).all()):
                raise CommError(f"guard page of the symmetric block at offset {off} "
                                f"({nbytes} bytes) was overwritten")

    def named(self, name: str, nbytes: int) -> SymmBlock:
        """Persistent block keyed by name; re-allocated (collectively) when it must grow."""
        b = self._named.get(name)
        if b is None or b.nbytes < nbytes:
            b = self.alloc(max(nbytes, 2 * b.nbytes if b else nbytes))
            self._named[name] = b
        return b

    def empty(self, shape, dtype=torch.bfloat16):
        """Symmetric tensor (collective).  Returns (tensor, block)."""
        n = 1
        for s in shape:
            n *= int(s)
        blk = self.alloc(n * torch.empty((), dtype=dtype).element_size())
        return blk.view(dtype, shape), blk

    def find_block(self, t: torch.Tensor):
        """(peer_ptrs, mc_ptr) if `t` lies inside the symmetric heap, else None."""
        p = t.data_ptr()
        for seg in self._segments:
            if seg["local"] <= p < seg["local"] + seg["nbytes"]:
                off = p - seg["local"]
                return [q + off for q in seg["peers"]], (seg["mc"] + off) if seg["mc"] else 0
        return None

    # --------------------------------------------------------------------- status
    def status_word(self) -> int:
        return int(self._status_host[0])

    def check_status(self, sync: bool = True):
        """Raises if a kernel recorded a time-out; clears the word."""
        if sync:
            torch.cuda.synchronize(self.device)
        w = self.status_word()
        if w != 0:
            self._status_host[0] = 0
            raise CommError(f"rank {self.rank}: device reported: {N.decode_status(w)}")

    def reset_sync_state(self):
        """After an error: zero pads and epochs on every rank (collective, host barriers)."""
        torch.cuda.synchronize(self.device)
        self.host_barrier()
        self.pad.local.zero_()
        self.epoch.zero_()
        self._status_host[0] = 0
        torch.cuda.synchronize(self.device)
        self.host_barrier()

    def close(self):
        if self._closed:
            return
        self._closed = True
        try:
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                self.host_barrier(10000)
        except Exception:
            pass
        for seg in self._segments:
            if seg.get("handle") is not None:
                self.lib.cb_symm_segment_destroy(seg["handle"])
            elif seg.get("ipc"):
                for r, q in enumerate(seg["peers"]):
                    if r != self.rank:
                        self.lib.cb_ipc_close(C.c_void_p(q))
                self.lib.cb_ipc_free(C.c_void_p(seg["local"]))
        self._segments = []
        if self._broker.value:
            self.lib.cb_broker_destroy(self._broker)
            self._broker = C.c_void_p(0)
        if self._status_host_ptr.value:
            self.lib.cb_mapped_free(self._status_host_ptr)
            self._status_host_ptr = C.c_void_p(0)


class EmuContext(_ContextBase):
    """``world`` virtual ranks on one GPU (single process, single launch per collective)."""

    def __init__(self, world: int, device: torch.device | None = None, timeout_s: float = 2.0):
        self.lib = N.load()
        if world not in (1, 2, 4, 8):
            raise CommError("world must be 1, 2, 4 or 8")
        self.world = world
        self.rank = 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.timeout_ns = int(timeout_s * 1e9)
        self.has_multicast = False
        self.pads = [torch.zeros(N.PAD_WORDS, dtype=torch.int32, device=self.device)
                     for _ in range(world)]
        self.epochs = [torch.zeros(N.PAD_CHANNELS, dtype=torch.int32, device=self.device)
                       for _ in range(world)]
        self.status = torch.zeros(world * 16, dtype=torch.int32, device=self.device)
        pad_ptrs = [p.data_ptr() for p in self.pads]
        self.comms = [self._make_comm(r, pad_ptrs, 0, self.epochs[r].data_ptr(),
                                      self.status.data_ptr() + 64 * r) for r in range(world)]

    def alloc(self, nbytes: int) -> list[torch.Tensor]:
        """One uint8 buffer per virtual rank (the 'symmetric' block)."""
        nbytes = (max(int(nbytes), 16) + 15) // 16 * 16
        return [torch.zeros(nbytes, dtype=torch.uint8, device=self.device) for _ in range(self.world)]

    def args_table(self, per_rank_args: list[N.CollArgs]) -> torch.Tensor:
        """Copies the per-rank argument blocks into device memory for an emulated launch."""
        sz = C.sizeof(N.CollArgs)
        raw = bytearray()
        for a in per_rank_args:
            raw += bytes(a)
        host = torch.frombuffer(raw, dtype=torch.uint8).clone()
        assert host.numel() == sz * len(per_rank_args)
        return host.to(self.device)

    def status_words(self) -> list[int]:
        torch.cuda.synchronize(self.device)
        s = self.status.cpu().view(self.world, 16)[:, 0].tolist()
        return [int(x) & 0xFFFFFFFF for x in s]

    def check_status(self):
        for r, w in enumerate(self.status_words()):
            if w != 0:
                self.status.zero_()
                raise CommError(f"virtual rank {r}: device reported: {N.decode_status(w)}")
