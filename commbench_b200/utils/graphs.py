"""CUDA-graph helpers for launch-bound inner loops.

The collective and fused kernels of this package keep their sequencing state on the device
(epoch counters in the signal pad, call counters of the fused ops), and their host wrappers pass
the same pointers on every call, so a captured launch can be replayed any number of times: each
replay advances the device-side epoch exactly as a fresh launch would.  Capturing removes the
Python / ctypes / launch overhead that dominates small messages (the reference times its
one-shot all-reduce the same way,
datasets/example105_sglang_custom_all_reduce_one_shot_hard/nv/empty_sglang_custom_all_reduce_one_shot.cu).

Every rank must capture and replay the same sequence.
"""
from __future__ import annotations

import torch


def capture(fn, repeat: int = 1, warmup: int = 3, stream: torch.cuda.Stream | None = None):
    """Runs ``fn`` ``warmup`` times eagerly (lazy initialisation, first-use attributes), then
    records ``repeat`` back-to-back calls of it into a graph.  Returns the graph; ``replay()``
    it on any stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = stream or torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
            for _ in range(repeat):
                fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    return g


def time_graphed(fn, calls_per_graph: int = 20, replays: int = 5, warmup: int = 3) -> float:
    """Milliseconds per call of ``fn`` when ``calls_per_graph`` calls are replayed as one graph
    (maximum over ranks when a process group is up)."""
    import torch.distributed as dist

    g = capture(fn, calls_per_graph, warmup)
    g.replay()
    torch.cuda.synchronize()
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    if multi:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / (replays * calls_per_graph)
    if multi:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms
