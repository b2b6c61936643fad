"""Data parallelism on the symmetric heap: bucketed gradient all-reduce (DDP style) and
sharded gradients / parameters (ZeRO style: reduce-scatter of gradients, all-gather of
parameters).

Gradients live in flat symmetric buckets from the start - each parameter's ``.grad`` is a view
into its bucket - so the collective runs in place on memory the peers can already reach (NVLS
``multimem.ld_reduce`` / ``multimem.st`` when bound, two-shot otherwise): no flatten / unflatten
copies and one launch per bucket.

The reference ships these as stand-alone primitives only: all-reduce
(datasets/example022_torch_distributed_nccl_allreduce, example048_thunderkitten_all_reduce_easy),
reduce-scatter + all-gather "ZeRO" all-reduce
(datasets/example031_msclpp_allreduce_rsag_zero_easy/empty_mscclpp_allreduce_easy.cu:1-50),
reduce-scatter (example023, example050) and all-gather (example021, example046).
"""
from __future__ import annotations

import torch

from ..ops import collectives as coll
from ..runtime.context import CommContext, CommError


class GradBuckets:
    """Flat symmetric gradient buckets for a list of parameters of one dtype per bucket."""

    def __init__(self, ctx: CommContext, params, bucket_bytes: int = 64 << 20):
        self.ctx = ctx
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise CommError("GradBuckets: no trainable parameters")
        self.buckets: list[torch.Tensor] = []
        self.views: list[list[tuple[torch.nn.Parameter, int, int]]] = []
        by_dtype: dict[torch.dtype, list] = {}
        for p in self.params:
            by_dtype.setdefault(p.dtype, []).append(p)
        for dtype, ps in by_dtype.items():
            esz = torch.empty((), dtype=dtype).element_size()
            cur, cur_n = [], 0
            for p in ps + [None]:
                n = 0 if p is None else (p.numel() + 7) // 8 * 8      # 16-byte aligned slots
                if p is None or (cur and (cur_n + n) * esz > bucket_bytes):
                    if cur:
                        # Padded so the bucket splits evenly over the ranks in 16-byte units.
                        unit = ctx.world * (16 // esz)
                        total = (cur_n + unit - 1) // unit * unit
                        flat, _ = ctx.empty((total,), dtype)
                        flat.zero_()
                        off, entries = 0, []
                        for q in cur:
                            q.grad = flat[off:off + q.numel()].view_as(q)
                            entries.append((q, off, q.numel()))
                            off += (q.numel() + 7) // 8 * 8
                        self.buckets.append(flat)
                        self.views.append(entries)
                    cur, cur_n = [], 0
                if p is not None:
                    cur.append(p)
                    cur_n += n

    def zero_grad(self):
        for b in self.buckets:
            b.zero_()

    def all_reduce(self, average: bool = True, algo: str = "auto"):
        """Sums (or averages) every gradient over the ranks, in place."""
        for b in self.buckets:
            coll.all_reduce(self.ctx, b, algo=algo)
            if average and self.ctx.world > 1:
                b.mul_(1.0 / self.ctx.world)

    # ------------------------------------------------------------------ ZeRO-style sharding
    def shard_range(self, bucket: int) -> tuple[int, int]:
        n = self.buckets[bucket].numel() // self.ctx.world
        return self.ctx.rank * n, (self.ctx.rank + 1) * n

    def reduce_scatter(self, average: bool = True) -> list[torch.Tensor]:
        """Each rank receives the reduced gradients of ITS slice of every bucket."""
        out = []
        for b in self.buckets:
            g = coll.reduce_scatter(self.ctx, b.view(self.ctx.world, -1))
            g = g.view(-1)
            if average and self.ctx.world > 1:
                g.mul_(1.0 / self.ctx.world)
            out.append(g)
        return out


class ShardedParams:
    """Flat parameter buckets whose slices are owned by different ranks: the owner updates its
    slice, ``all_gather`` republishes the whole bucket (ZeRO stage 1/2 parameter refresh)."""

    def __init__(self, ctx: CommContext, params):
        self.ctx = ctx
        self.params = list(params)
        dtype = self.params[0].dtype
        if any(p.dtype != dtype for p in self.params):
            raise CommError("ShardedParams: one dtype per group")
        esz = torch.empty((), dtype=dtype).element_size()
        unit = ctx.world * (16 // esz)
        n = sum((p.numel() + 7) // 8 * 8 for p in self.params)
        self.total = (n + unit - 1) // unit * unit
        self.flat, _ = ctx.empty((self.total,), dtype)
        self.flat.zero_()
        off = 0
        with torch.no_grad():
            for p in self.params:
                view = self.flat[off:off + p.numel()].view_as(p)
                view.copy_(p)
                p.data = view                       # the module now computes on the bucket
                off += (p.numel() + 7) // 8 * 8

    def local_shard(self) -> torch.Tensor:
        n = self.total // self.ctx.world
        return self.flat[self.ctx.rank * n:(self.ctx.rank + 1) * n]

    def all_gather(self):
        """Publishes every rank's updated slice to all ranks (pushed straight into the peers'
        copies of the bucket)."""
        if self.ctx.world > 1:
            shard = self.local_shard().clone()
            coll.all_gather(self.ctx, shard, out=self.flat)
