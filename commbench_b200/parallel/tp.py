"""Tensor parallelism: column- and row-parallel linear layers whose collective is fused into
the GEMM kernel (inference / forward path).

* ``ColumnParallelLinear``: activations are sharded by rows (sequence parallel) across ranks,
  the weight by output features.  ``y = all_gather_rows(x_local) @ W_local^T`` in one kernel
  (all-gather -> GEMM).
* ``RowParallelLinear``: the weight is sharded by input features; the partial products are
  summed across ranks inside the GEMM epilogue, either scattered by rows
  (GEMM -> reduce-scatter, sequence parallel output) or replicated (GEMM -> all-reduce, the
  decode path).

Sharding conventions follow the reference's fused examples: activation rows M/W per rank and
N/W weight rows per rank for all-gather + GEMM
(datasets/example051_thunderkitten_ag_gemm_easy/nv/empty_thunderkitten_ag_gemm.cu:470-478), K
sharded with rows scattered for GEMM + reduce-scatter
(datasets/example054_thunderkitten_gemm_rs_easy/nv/empty_thunderkitten_gemm_rs.cu:450-460), K
sharded with a replicated result for GEMM + all-reduce
(datasets/example053_thunderkitten_gemm_ar_easy/nv/empty_thunderkitten_gemm_ar.cu:491-499).
"""
from __future__ import annotations

import torch

from ..ops.gemm import gemm
from ..ops.tp import AgGemm, GemmAr, GemmRs


def _init_weight(out_f: int, in_f: int, device, seed: int) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(out_f, in_f, device=device, generator=g) * 0.02).bfloat16()


class ColumnParallelLinear:
    """``in_features`` -> ``out_features`` with the output features split over the ranks."""

    def __init__(self, ctx, in_features: int, out_features: int, max_tokens: int, seed: int = 0,
                 weight: torch.Tensor | None = None):
        self.ctx, self.world = ctx, ctx.world
        if out_features % ctx.world or max_tokens % ctx.world:
            raise ValueError("out_features and max_tokens must divide by the world size")
        self.out_local = out_features // ctx.world
        self.weight = weight if weight is not None else \
            _init_weight(self.out_local, in_features, ctx.device, seed * 1000 + ctx.rank)
        self._op = AgGemm(ctx, max_tokens, in_features) if ctx.world > 1 else None

    def __call__(self, x_local: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """``x_local`` [tokens / W, in] -> [tokens, out / W]."""
        if self._op is None:
            return gemm(x_local, self.weight, out=out)
        return self._op(x_local, self.weight, out=out)


class RowParallelLinear:
    """``in_features`` (split over the ranks) -> ``out_features``; ``scatter_rows=True`` returns
    this rank's rows of the sum, otherwise every rank gets the whole sum."""

    def __init__(self, ctx, in_features: int, out_features: int, max_tokens: int,
                 scatter_rows: bool = True, seed: int = 1, weight: torch.Tensor | None = None):
        self.ctx, self.world, self.scatter_rows = ctx, ctx.world, scatter_rows
        if in_features % ctx.world:
            raise ValueError("in_features must divide by the world size")
        self.in_local = in_features // ctx.world
        self.weight = weight if weight is not None else \
            _init_weight(out_features, self.in_local, ctx.device, seed * 1000 + ctx.rank)
        if ctx.world == 1:
            self._op = None
        elif scatter_rows:
            self._op = GemmRs(ctx, max_tokens, out_features)
        else:
            self._op = GemmAr(ctx, max_tokens, out_features)

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """``x`` [tokens, in / W] -> [tokens / W, out] (scatter_rows) or [tokens, out]."""
        if self._op is None:
            return gemm(x, self.weight, out=out)
        return self._op(x, self.weight, out=out)
