"""Tracing helpers: NVTX ranges, per-kernel device times out of a profiler trace, and a span
recorder that writes a Chrome trace (``chrome://tracing`` / Perfetto JSON).

The reference has no tracing layer; its one profiler hook extracts the duration of named kernels
from a torch-profiler trace (``bench_kineto(fn, kernel_names=..., num_tests=10)`` in
datasets/example080_deepep_jit_dispatch_payload/nv/build_and_run.py:751-759) - that is
:func:`kernel_times` here.  NVTX ranges (off unless ``CB200_NVTX=1``) make the ops show up by name
in an external profiler's timeline; :class:`SpanRecorder` gives a timeline without one.
"""
from __future__ import annotations

import contextlib
import functools
import json
import os
import time

import torch


def nvtx_enabled() -> bool:
    from ..config import get_config

    return bool(get_config().nvtx) and torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str, force: bool = False):
    """Pushes an NVTX range around the block when tracing is on (or ``force``); free otherwise."""
    on = (force and torch.cuda.is_available()) or nvtx_enabled()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def traced(name: str | None = None):
    """Decorator form of :func:`nvtx_range`."""
    def wrap(fn):
        label = name or fn.__qualname__

        @functools.wraps(fn)
        def inner(*a, **kw):
            with nvtx_range(label):
                return fn(*a, **kw)
        return inner
    return wrap


# ------------------------------------------------------------ kernel times from a profiler trace
def aggregate_kernel_events(events, names=None) -> dict:
    """``events``: iterable of (kernel name, duration in microseconds).  Returns
    ``{name: {"calls", "total_us", "mean_us", "min_us", "max_us"}}``; with ``names`` given, keys
    are those substrings and every kernel whose name contains one is counted under it."""
    out: dict[str, dict] = {}
    for kname, dur in events:
        keys = [kname] if names is None else [n for n in names if n in kname]
        for k in keys:
            s = out.setdefault(k, {"calls": 0, "total_us": 0.0, "min_us": float("inf"), "max_us": 0.0})
            s["calls"] += 1
            s["total_us"] += float(dur)
            s["min_us"] = min(s["min_us"], float(dur))
            s["max_us"] = max(s["max_us"], float(dur))
    for s in out.values():
        s["mean_us"] = s["total_us"] / s["calls"]
    return out


def kernel_times(fn, names=None, iters: int = 10, warmup: int = 3, barrier=None) -> dict:
    """Runs ``fn`` ``iters`` times under the torch profiler and returns the device time of every
    kernel (or of those whose name contains one of ``names``), aggregated over the calls.
    ``barrier`` (a callable) runs before every call so that ranks start together.  The profiler
    adds overhead to the host side; kernel durations are the device's own."""
    from torch.profiler import ProfilerActivity, profile

    for _ in range(warmup):
        fn()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    with profile(activities=acts) as prof:
        for _ in range(iters):
            if barrier is not None:
                barrier()
            fn()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
    events = []
    for ev in prof.events():
        is_kernel = getattr(ev, "device_type", None) is not None and "cuda" in str(ev.device_type).lower()
        if torch.cuda.is_available() and not is_kernel:
            continue
        dur = getattr(ev, "device_time", None)
        if not dur:
            dur = getattr(ev, "cpu_time", 0.0)
        events.append((ev.name, dur))
    return aggregate_kernel_events(events, names)


# ------------------------------------------------------------------------- span recorder
class SpanRecorder:
    """Named spans on one stream, timed with CUDA events (host clock without a GPU), exported as a
    Chrome trace.  Spans may nest.  Nothing synchronises until :meth:`spans` / :meth:`export`."""

    def __init__(self, process_name: str | None = None, rank: int | None = None):
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.process_name = process_name or f"rank {self.rank}"
        self.cuda = torch.cuda.is_available()
        self._open: list = []
        self._done: list = []
        self._origin = self._stamp()

    def _stamp(self):
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter()

    @contextlib.contextmanager
    def span(self, name: str, **args):
        start = self._stamp()
        depth = len(self._open)
        self._open.append(name)
        try:
            with nvtx_range(name):
                yield
        finally:
            self._open.pop()
            self._done.append((name, depth, start, self._stamp(), args))

    def _us(self, a, b) -> float:
        return a.elapsed_time(b) * 1e3 if self.cuda else (b - a) * 1e6

    def spans(self) -> list[dict]:
        """[{name, depth, start_us, dur_us, args}] in start order (synchronises the device)."""
        if self.cuda:
            torch.cuda.synchronize()
        rows = [{"name": n, "depth": d, "start_us": self._us(self._origin, s), "dur_us": self._us(s, e),
                 "args": a} for n, d, s, e, a in self._done]
        return sorted(rows, key=lambda r: (r["start_us"], r["depth"]))

    def export(self, path: str) -> str:
        events = [{"name": "process_name", "ph": "M", "pid": self.rank, "args": {"name": self.process_name}}]
        for r in self.spans():
            events.append({"name": r["name"], "ph": "X", "pid": self.rank, "tid": r["depth"],
                           "ts": r["start_us"], "dur": r["dur_us"], "args": r["args"]})
        os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
        with open(path, "w") as f:
            json.dump({"traceEvents": events, "displayTimeUnit": "ns"}, f)
        return path


def merge_chrome_traces(paths: list[str], out: str) -> str:
    """One trace file out of the per-rank files (each rank is a process row)."""
    events = []
    for p in paths:
        with open(p) as f:
            events += json.load(f)["traceEvents"]
    with open(out, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ns"}, f)
    return out
