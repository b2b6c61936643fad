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
