"""What the multi-GPU task programs share: rank set-up, the "not enough GPUs" exit, device
timing with the maximum over ranks, and the one JSON line a task prints.

The reference's multi-GPU examples print ``"Correctness":"SKIP"`` and exit 0 when the machine
has fewer GPUs than ranks (datasets/example017_intranode_gpu_barrier/nv/
empty_intranode_gpu_barrier.cu:224-229); :func:`start` does the same before any process
group or symmetric heap exists, so a task is safe to launch anywhere.
"""
from __future__ import annotations

import json
import os
import sys


def _emit(obj: dict) -> None:
    print(json.dumps(obj), flush=True)


def skip(reason: str) -> None:
    """Rank 0 prints the SKIP line; every rank exits 0."""
    if int(os.environ.get("RANK", "0")) == 0:
        _emit({"Correctness": "SKIP", "reason": reason, "data_size_unit": "MB", "latency_unit": "us",
               "throughput_unit": "GB/s", "metrics": []})
    sys.exit(0)


_ACTIVE: list = []


class TaskRun:
    """One rank of a task.  ``ctx`` is the symmetric-memory context (created on first use)."""

    def __init__(self, heap_mb: int):
        _ACTIVE.append(self)
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        self.dev = torch.device("cuda", local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self._heap_mb = heap_mb
        self._ctx = None

    @property
    def ctx(self):
        if self._ctx is None:
            from ..runtime.context import CommContext

            self._ctx = CommContext(heap_bytes=self._heap_mb << 20)
        return self._ctx

    def sync(self) -> None:
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def timed_us(self, fn, iters: int = 10, warmup: int = 3) -> float:
        """Mean device time of ``fn`` in microseconds (CUDA events), maximum over ranks."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        self.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        self.sync()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_ok(self, flag: bool) -> bool:
        t = self.torch.tensor([1 if flag else 0], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item())

    def teardown(self) -> None:
        """Frees the symmetric heap (unbinding it from the multicast object) and the process
        group, in that order, after the device went idle.  Idempotent."""
        if self in _ACTIVE:
            _ACTIVE.remove(self)
        try:
            self.torch.cuda.synchronize()
        except Exception:
            pass
        if self._ctx is not None:
            ctx, self._ctx = self._ctx, None
            ctx.close()
        if self.world > 1 and self.dist.is_initialized():
            self.dist.destroy_process_group()

    def finish(self, ok: bool, rows: list[dict], **extra) -> None:
        """Prints the result line on rank 0 and tears everything down."""
        ok = self.all_ok(bool(ok) and len(rows) > 0)
        if self._ctx is not None:
            try:
                self._ctx.check_status()
            except Exception as ex:  # a device-side time-out fails the task, it does not hang it
                ok = False
                extra["device_status"] = str(ex)
        if self.rank == 0:
            _emit({"throughput_unit": "GB/s", **extra,
                   "Correctness": "PASS" if ok else "FAIL", "data_size_unit": "MB",
                   "latency_unit": "us", "metrics": rows})
        self.teardown()


def guarded(body) -> None:
    """Runs a task's ``main``.  An exception (an unfilled skeleton raises NotImplementedError on
    every rank at the same point) still ends in an orderly teardown - no rank exits while its
    memory is bound to a multicast object - then rank 0 prints a FAIL line and the exit code is 1."""
    try:
        body()
    except SystemExit:
        raise
    except BaseException as ex:  # noqa: BLE001 - reported, then the process exits non-zero
        for run in list(_ACTIVE):
            try:
                run.teardown()
            except Exception:
                pass
        if int(os.environ.get("RANK", "0")) == 0:
            _emit({"Correctness": "FAIL", "error": f"{type(ex).__name__}: {ex}"[:400],
                   "metrics": []})
        sys.exit(1)


def start(min_world: int = 2, heap_mb: int = 512, need_multicast: bool = False) -> TaskRun:
    """Set-up of a GPU task; exits with the SKIP line when the machine cannot run it."""
    try:
        import torch
    except ImportError:
        skip("PyTorch is not installed")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        skip("no CUDA device")
    if world < min_world:
        skip(f"needs {min_world} ranks, launched with {world}")
    if torch.cuda.device_count() < world:
        skip(f"needs {world} GPUs, found {torch.cuda.device_count()}")
    from .. import _native

    if not _native.available():
        skip("the native library is not built")
    run = TaskRun(heap_mb)
    if need_multicast and not run.ctx.has_multicast:
        run.teardown()
        skip("no NVLink multicast object could be bound")
    return run
