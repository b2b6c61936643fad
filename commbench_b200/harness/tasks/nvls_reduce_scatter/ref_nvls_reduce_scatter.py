"""Reduce-scatter of a symmetric [W * rows, 256] bf16 tensor: rank r receives the sum over ranks
of row block r, taken with ``multimem.ld_reduce`` (the switch adds the W copies) straight into a
local output.  Prints one JSON object.

Same exercise as the reference's datasets/example050_thunderkitten_reduce_scatter_easy (TK
reduce-scatter, :64-95).

Launched as: torchrun --nproc-per-node W ref_nvls_reduce_scatter.py
"""
import torch
import torch.distributed as dist

from commbench_b200.harness import tasklib
from commbench_b200.ops import collectives as coll

SIZES_MB = (2, 16, 64)


class NvlsReduceScatter:
    def __init__(self, run: tasklib.TaskRun, max_bytes: int):
        self.ctx, self.W = run.ctx, run.world
        rows = max_bytes // 512 // self.W * self.W
        # --- solution: the INPUT lives in the symmetric heap; a plain local tensor takes the result
        self.x, _ = self.ctx.empty((rows, 256), torch.bfloat16)
        self.out = torch.empty(rows // self.W, 256, device=run.dev, dtype=torch.bfloat16)
        # --- end solution

    def run(self, rows: int) -> torch.Tensor:
        """Sum over ranks of row block `rank` of the first `rows` rows of self.x."""
        # --- solution: one launch; use_nvls=True asks for the in-switch reduction
        return coll.reduce_scatter(self.ctx, self.x[:rows], out=self.out[: rows // self.W],
                                   use_nvls=True)
        # --- end solution


def main():
    run = tasklib.start(min_world=2, heap_mb=256, need_multicast=True)
    op = NvlsReduceScatter(run, max(SIZES_MB) << 20)
    ok, rows_out = True, []
    for mb in SIZES_MB:
        rows = (mb << 20) // 512 // run.world * run.world
        g = torch.Generator(device=run.dev).manual_seed(31 + run.rank)
        x = (torch.rand(rows, 256, device=run.dev, generator=g) * 2 - 1).bfloat16()
        ref = torch.empty(rows // run.world, 256, device=run.dev, dtype=torch.float32)
        dist.reduce_scatter_tensor(ref, x.float())
        op.x[:rows].copy_(x)
        run.sync()
        y = op.run(rows)
        torch.cuda.synchronize()
        ok &= y is not None and tuple(y.shape) == (rows // run.world, 256)
        ok &= bool(((y.float() - ref).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))).item())
        us = run.timed_us(lambda: op.run(rows))
        bus = (run.world - 1) / run.world * (rows * 512) / (us * 1e-6) / 1e9
        rows_out.append({"data_size": rows * 512 / 2**20, "latency_avg": us, "throughput_avg": bus})
    run.finish(ok, rows_out)


if __name__ == "__main__":
    tasklib.guarded(main)
