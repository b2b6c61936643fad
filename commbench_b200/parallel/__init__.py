"""Parallelism strategies as components built on the ops:

* ``dp``: bucketed gradient all-reduce and ZeRO-style sharded gradients / parameters
* ``tp``: column- / row-parallel linear layers with the collective fused into the GEMM
* ``pp``: pipeline-stage hand-off (tensors and tensor dicts over NCCL p2p on a side stream)
* ``ep``: expert-parallel MoE feed-forward (fp8 dispatch, grouped GEMMs, combine)
* ``cp``: context-parallel attention (ring with K/V prefetch, Ulysses head exchange)
"""
from . import cp, dp, ep, pp, tp  # noqa: F401
