"""Device-side timing helpers: CUDA events on the launching stream, warm-up first, maximum over
ranks for anything multi-GPU (the timing method of every harness entry)."""
from __future__ import annotations

import torch


def time_ms(fn, iters: int = 10, warmup: int = 3, group_max: bool = True) -> float:
    """Milliseconds per call of ``fn``; with an initialised process group the maximum over ranks."""
    import torch.distributed as dist

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    multi = group_max and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    if multi:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    if multi:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def latency_stats(samples) -> dict:
    """``{count, min, avg, p50, p90, p99, max}`` of a list of per-call times (any unit); the
    percentile is the nearest-rank one, so every reported value is a value that was measured.
    The reference's queue benchmarks print the same set
    (datasets/example003_fifo_device2host/empty_fifo_test_unified.cu:656-669)."""
    xs = sorted(float(x) for x in samples)
    if not xs:
        return {"count": 0, "min": None, "avg": None, "p50": None, "p90": None, "p99": None, "max": None}

    def rank(p: int) -> float:
        k = -(-p * len(xs) // 100)                    # ceil(p / 100 * n): nearest-rank percentile
        return xs[min(len(xs), max(1, k)) - 1]

    return {"count": len(xs), "min": xs[0], "avg": sum(xs) / len(xs), "p50": rank(50), "p90": rank(90),
            "p99": rank(99), "max": xs[-1]}


def time_each_ms(fn, iters: int = 100, warmup: int = 3) -> list[float]:
    """Per-call device times: one CUDA event pair per call (adds an event record between calls,
    so use ``time_ms`` for throughput and this for the latency distribution)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
    evs[0].record()
    for i in range(iters):
        fn()
        evs[i + 1].record()
    torch.cuda.synchronize()
    return [evs[i].elapsed_time(evs[i + 1]) for i in range(iters)]


class DeviceTimer:
    """``with DeviceTimer() as t: ...`` then ``t.ms`` (synchronises on exit)."""

    def __enter__(self):
        self._e0, self._e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self._e0.record()
        return self

    def __exit__(self, *exc):
        self._e1.record()
        torch.cuda.synchronize()
        self.ms = self._e0.elapsed_time(self._e1)
