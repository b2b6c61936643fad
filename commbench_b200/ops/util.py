"""Utilities under the collectives: GPU<->CPU FIFOs, shared-memory object broadcast,
bandwidth / latency probes, device attributes, CUDA-IPC tensor hand-off.

Reference counterparts: datasets/example003_fifo_device2host (D2H trigger FIFO + proxy thread),
datasets/example005_fifo_host2device (H2D task FIFO + persistent kernel),
datasets/example100_vllm_shm_broadcast_object (shm MessageQueue), datasets/example072...077 and
example094 (probes), datasets/example010_list_gpu_attributes, datasets/example088_vllm_ipc_weight_transfer_engine
and datasets/example012_gpu_ipc_comm_with_NVLink (IPC hand-off).
"""
from __future__ import annotations

import ctypes as C
import json
import pickle

import torch

from .. import _native as N


class UtilError(RuntimeError):
    pass


# --------------------------------------------------------------------- D2H FIFO
class D2HFifo:
    """Device-to-host trigger queue with a host proxy thread."""

    def __init__(self, size: int = 512):
        self.lib = N.load()
        self._h = C.c_void_p(0)
        N.check(self.lib.cb_d2h_fifo_create(size, C.byref(self._h)), "cb_d2h_fifo_create")
        self.size = size

    def start_proxy(self):
        N.check(self.lib.cb_d2h_fifo_proxy_start(self._h), "proxy_start")

    def stop_proxy(self):
        popped, checksum, span = C.c_ulonglong(0), C.c_ulonglong(0), C.c_ulonglong(0)
        N.check(self.lib.cb_d2h_fifo_proxy_stop(self._h, C.byref(popped), C.byref(checksum),
                                                C.byref(span)), "proxy_stop")
        return popped.value, checksum.value, span.value

    def popped(self) -> int:
        self.lib.cb_d2h_fifo_popped.restype = C.c_ulonglong
        return int(self.lib.cb_d2h_fifo_popped(self._h))

    def poll(self):
        fst, snd = C.c_ulonglong(0), C.c_ulonglong(0)
        if self.lib.cb_d2h_fifo_poll(self._h, C.byref(fst), C.byref(snd)):
            return fst.value, snd.value
        return None

    def pop(self):
        self.lib.cb_d2h_fifo_pop(self._h)

    def push_test(self, blocks: int, threads: int, per_thread: int, timeout_s: float = 2.0,
                  status: torch.Tensor | None = None, push_ns: torch.Tensor | None = None):
        """Launches the kernel in which every thread pushes `per_thread` triggers (fst = 1-based id)."""
        N.check(self.lib.cb_d2h_fifo_push_test(self._h, blocks, threads, per_thread,
                                               C.c_ulonglong(int(timeout_s * 1e9)), N.ptr(status),
                                               N.ptr(push_ns), N.stream_ptr()), "push_test")

    def close(self):
        if self._h.value:
            self.lib.cb_d2h_fifo_destroy(self._h)
            self._h = C.c_void_p(0)


# --------------------------------------------------------------------- H2D FIFO
class H2DFifo:
    """Host-to-device task queue consumed by a persistent kernel."""

    def __init__(self, size: int = 64):
        self.lib = N.load()
        self._h = C.c_void_p(0)
        N.check(self.lib.cb_h2d_fifo_create(size, C.byref(self._h)), "cb_h2d_fifo_create")
        self.size = size

    def launch_consumer(self, expect: int, timeout_s: float = 2.0,
                        status: torch.Tensor | None = None, stream=None) -> torch.Tensor:
        """Starts the consumer for `expect` items; returns the [expect, 2] result tensor
        (value, pop time in ns) that is complete once the stream has drained."""
        res = torch.zeros(expect, 2, dtype=torch.int64, device="cuda")
        N.check(self.lib.cb_h2d_fifo_launch_consumer(self._h, C.c_ulonglong(expect), N.ptr(res),
                                                     C.c_ulonglong(int(timeout_s * 1e9)),
                                                     N.ptr(status), N.stream_ptr(stream)),
                "launch_consumer")
        return res

    def push(self, value: int, timeout_ms: int = 2000):
        rc = self.lib.cb_h2d_fifo_push(self._h, C.c_ulonglong(value), timeout_ms)
        if rc != 0:
            raise UtilError(f"h2d push failed: {N.last_error()}")

    def close(self):
        if self._h.value:
            self.lib.cb_h2d_fifo_destroy(self._h)
            self._h = C.c_void_p(0)


# -------------------------------------------------------- shm object broadcast
class ShmBroadcast:
    """One writer, N readers on the same host; objects are pickled."""

    def __init__(self, name: str, n_readers: int, reader_index: int | None = None,
                 nslots: int = 16, slot_bytes: int = 1 << 16, timeout_ms: int = 10000):
        self.lib = N.load()
        self._h = C.c_void_p(0)
        self.is_writer = reader_index is None
        if self.is_writer:
            N.check(self.lib.cb_shmq_create(name.encode(), n_readers, nslots, slot_bytes,
                                            C.byref(self._h)), "cb_shmq_create")
        else:
            N.check(self.lib.cb_shmq_open(name.encode(), reader_index, timeout_ms,
                                          C.byref(self._h)), "cb_shmq_open")
        self._buf = C.create_string_buffer(1 << 20)

    def broadcast_object(self, obj, timeout_ms: int = 10000):
        data = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
        rc = self.lib.cb_shmq_write(self._h, data, C.c_longlong(len(data)), timeout_ms)
        if rc != 0:
            raise UtilError(f"shm broadcast failed: {N.last_error()}")

    def dequeue(self, timeout_ms: int = 10000):
        n = C.c_longlong(0)
        while True:
            rc = self.lib.cb_shmq_read(self._h, self._buf, C.c_longlong(len(self._buf)),
                                       C.byref(n), timeout_ms)
            if rc == -3:
                self._buf = C.create_string_buffer(len(self._buf) * 4)
                raise UtilError("message larger than the receive buffer (buffer grown; resend)")
            if rc == -2:
                raise TimeoutError(N.last_error())
            if rc != 0:
                raise UtilError(N.last_error())
            return pickle.loads(self._buf.raw[:n.value])

    def close(self):
        if self._h.value:
            self.lib.cb_shmq_close(self._h)
            self._h = C.c_void_p(0)


# ------------------------------------------------------------------------ probes
_ABS_MEAN_SCRATCH: dict = {}


def abs_mean(x: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """``mean(|x|)`` of a bf16 CUDA tensor as a one-element fp32 tensor, in ONE pass over ``x``
    (``x.float().abs().mean()`` writes and re-reads two fp32 copies).  Falls back to that
    expression for other dtypes, unaligned or non-contiguous inputs."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and
            x.numel() % 8 == 0 and x.data_ptr() % 16 == 0 and x.numel() > 0):
        r = x.float().abs().mean().reshape(1)
        return r if out is None else out.copy_(r)
    lib = N.load()
    key = (x.device.index, (stream or torch.cuda.current_stream()).cuda_stream)
    scratch = _ABS_MEAN_SCRATCH.get(key)
    if scratch is None:
        scratch = _ABS_MEAN_SCRATCH[key] = torch.zeros(2, dtype=torch.int32, device=x.device)
    if out is None:
        out = torch.empty(1, dtype=torch.float32, device=x.device)
    rc = lib.cb_abs_mean_bf16(C.c_void_p(x.data_ptr()), C.c_longlong(x.numel()),
                              C.c_void_p(out.data_ptr()), C.c_void_p(scratch.data_ptr()),
                              N.stream_ptr(stream))
    if rc != 0:
        raise UtilError(f"abs_mean failed: {N.last_error()}")
    return out


def device_attributes(device: int = 0) -> dict:
    lib = N.load()
    buf = C.create_string_buffer(4096)
    n = lib.cb_probe_attributes_json(device, buf, len(buf))
    if n < 0:
        raise UtilError(f"attributes: {N.last_error()}")
    return json.loads(buf.value.decode())


def _time_ms(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def copy_bandwidth(dst_ptr: int, src_ptr: int, nbytes: int, width: int = 16, blocks: int = 592,
                   threads: int = 512, iters: int = 10, warmup: int = 3) -> float:
    """GB/s of a grid-stride copy kernel at the given vector width (4, 8 or 16 bytes)."""
    lib = N.load()

    def run():
        N.check(lib.cb_probe_copy(C.c_void_p(dst_ptr), C.c_void_p(src_ptr), C.c_longlong(nbytes),
                                  width, blocks, threads, N.stream_ptr()), "cb_probe_copy")
    ms = _time_ms(run, iters, warmup)
    return nbytes / ms / 1e6


def memcpy_bandwidth(dst: torch.Tensor, src: torch.Tensor, iters: int = 10, warmup: int = 3) -> float:
    """GB/s of the runtime's own copy (copy engine) between two tensors."""
    ms = _time_ms(lambda: dst.copy_(src, non_blocking=True), iters, warmup)
    return src.numel() * src.element_size() / ms / 1e6


def nanosleep_probe(request_ns: int, reps: int = 20) -> dict:
    lib = N.load()
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    N.check(lib.cb_probe_nanosleep(request_ns, reps, N.ptr(out), N.stream_ptr()), "nanosleep")
    torch.cuda.synchronize()
    measured, res = out.tolist()
    return {"request_ns": request_ns, "measured_ns": measured, "error_ns": measured - request_ns,
            "timer_resolution_ns": res}


def mbarrier_round_trip(threads: int = 128, iters: int = 4096) -> dict:
    lib = N.load()
    cyc = torch.zeros(1, dtype=torch.int64, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    N.check(lib.cb_probe_mbarrier(threads, iters, N.ptr(cyc), N.ptr(st), N.stream_ptr()), "mbarrier")
    torch.cuda.synchronize()
    if int(st.item()) != 0:
        raise UtilError("mbarrier probe timed out: " + N.decode_status(int(st.item()) & 0xFFFFFFFF))
    return {"threads": threads, "iters": iters, "cycles_per_iter": cyc.item() / iters}


def tma_stream_bandwidth(src: torch.Tensor, tile_bytes: int = 65536, stages: int = 3,
                         iters: int = 256, blocks: int = 148) -> float:
    """Aggregate GB/s of TMA bulk gmem->smem streaming (one producer thread per CTA)."""
    lib = N.load()
    sink = torch.zeros(blocks, dtype=torch.int64, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    nbytes = src.numel() * src.element_size()

    def run():
        N.check(lib.cb_probe_tma_stream(N.ptr(src), C.c_longlong(nbytes), tile_bytes, stages, iters,
                                        blocks, N.ptr(sink), N.ptr(st), N.stream_ptr()),
                "tma_stream")
    ms = _time_ms(run, 5, 2)
    if int(st.item()) != 0:
        raise UtilError("tma probe timed out")
    return blocks * iters * tile_bytes / ms / 1e6


# --------------------------------------------------------- CUDA-IPC tensor share
def ipc_export(t: torch.Tensor):
    """Picklable handle of a CUDA tensor for another process on the same host (the
    `reduce_tensor` hand-off of the reference's IPC weight transfer)."""
    from torch.multiprocessing.reductions import reduce_tensor

    fn, args = reduce_tensor(t)
    return (fn, args)


def ipc_import(handle) -> torch.Tensor:
    fn, args = handle
    return fn(*args)


# ------------------------------------------------------------- multi-GPU point-to-point probes
def pingpong_latency(ctx, rounds: int = 2000) -> float | None:
    """Round-trip time in microseconds of a one-word ping-pong between ranks 0 and 1 through
    peer memory (one warp per GPU, release store + bounded acquire wait).  Collective over the
    context; ranks above 1 only take part in the barriers and return ``None``
    (datasets/example073_GPU_p2p_pingpong_latency/nv/empty_p2p_pingpong_latency.cu:30-56)."""
    lib = N.load()
    blk = ctx.named("probe_pingpong", 256)
    word = blk.view(torch.int32, (64,))
    if not getattr(ctx, "_pingpong_ready", False):
        word.zero_()
        ctx._pingpong_ready = True
        torch.cuda.synchronize(ctx.device)
        ctx.host_barrier()
    base = int(word[1].item())                       # running value: the words only ever grow
    elapsed = torch.zeros(1, dtype=torch.int64, device=ctx.device)
    torch.cuda.synchronize(ctx.device)
    ctx.host_barrier()
    out = None
    if ctx.rank < 2 and ctx.world >= 2:
        peer = 1 - ctx.rank
        N.check(lib.cb_probe_pingpong(C.c_void_p(blk.peer_ptrs[ctx.rank]),
                                      C.c_void_p(blk.peer_ptrs[peer]), ctx.rank, rounds,
                                      C.c_uint(base), C.c_ulonglong(ctx.timeout_ns),
                                      C.c_void_p(ctx.comm.status), N.ptr(elapsed), N.stream_ptr()),
                "cb_probe_pingpong")
        torch.cuda.synchronize(ctx.device)
        ctx.check_status()
        out = elapsed.item() / rounds / 1e3
    word[1] = base + rounds
    torch.cuda.synchronize(ctx.device)
    ctx.host_barrier()
    return out


def peer_copy_bandwidth(ctx, nbytes: int, mode: str = "kernel", iters: int = 10, warmup: int = 3) -> float:
    """GB/s of pushing ``nbytes`` from this rank into the next rank's symmetric memory, with the
    16-byte copy kernel (``mode="kernel"``) or the copy engine (``mode="engine"``).  Every rank
    pushes at once (datasets/example074_GPU_p2p_d2d_bandwidth/nv/empty_p2p_d2d_bandwidth.cu:29-36,
    datasets/example001_gpu_comm_single_process/nv/empty_gpu_comm_single_process.cu)."""
    from ..runtime.context import tensor_from_ptr

    blk = ctx.named("probe_peer_copy", nbytes)
    src = torch.empty(nbytes, dtype=torch.uint8, device=ctx.device)
    src.fill_(ctx.rank + 1)
    peer = (ctx.rank + 1) % ctx.world
    dst_ptr = blk.peer_ptrs[peer]
    torch.cuda.synchronize(ctx.device)
    ctx.host_barrier()
    if mode == "kernel":
        gbs = copy_bandwidth(dst_ptr, src.data_ptr(), nbytes, 16, iters=iters, warmup=warmup)
    else:
        dst = tensor_from_ptr(dst_ptr, nbytes, ctx.device, owner=ctx)
        gbs = memcpy_bandwidth(dst, src, iters, warmup)
    torch.cuda.synchronize(ctx.device)
    ctx.host_barrier()
    got = int(blk.view(torch.uint8, (nbytes,))[nbytes - 1].item())
    if got != (ctx.rank - 1) % ctx.world + 1:
        raise UtilError(f"peer copy: expected the previous rank's pattern, found {got}")
    return gbs


def barrier_latency(ctx, iters: int = 1000, use_nvls: bool = False) -> float:
    """Microseconds per cross-GPU barrier, measured over ``iters`` back-to-back barriers inside
    one launch (datasets/example017_intranode_gpu_barrier/nv/empty_intranode_gpu_barrier.cu:114-125)."""
    from . import collectives as coll

    coll.barrier(ctx, 8, use_nvls)
    torch.cuda.synchronize(ctx.device)
    ctx.host_barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    coll.barrier(ctx, iters, use_nvls)
    e1.record()
    torch.cuda.synchronize(ctx.device)
    ctx.check_status()
    return e0.elapsed_time(e1) * 1e3 / iters
