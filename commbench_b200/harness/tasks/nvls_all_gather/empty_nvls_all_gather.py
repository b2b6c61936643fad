"""All-gather into a symmetric output with multicast stores: every rank writes its shard once,
to the multicast alias of the gathered tensor, and the NVSwitch replicates it to all ranks.
Prints one JSON object.

Same exercise as the reference's datasets/example046_thunderkitten_all_gather_easy (TK all-gather
with a multicast store per tile, :56-104).

Launched as: torchrun --nproc-per-node W ref_nvls_all_gather.py
"""
import torch
import torch.distributed as dist

from commbench_b200.harness import tasklib
from commbench_b200.ops import collectives as coll

SHARD_MB = (1, 8, 32)


class NvlsAllGather:
    """Gathered tensor [W * rows, 256] bf16 in symmetric memory; shards are ordinary tensors."""

    def __init__(self, run: tasklib.TaskRun, max_shard_bytes: int):
        self.ctx, self.W = run.ctx, run.world
        rows = max_shard_bytes // 512
        # TODO: the OUTPUT lives in the symmetric heap, W shards of `rows` rows
        raise NotImplementedError

    def run(self, shard: torch.Tensor) -> torch.Tensor:
        """Returns the gathered [W * shard_rows, 256] view of the symmetric output."""
        # TODO: push form of the all-gather - pass the symmetric view as `out`, force the
        #       multicast store (multicast=True): one multimem.st per 16-byte vector
        raise NotImplementedError


def main():
    run = tasklib.start(min_world=2, heap_mb=512, need_multicast=True)
    op = NvlsAllGather(run, max(SHARD_MB) << 20)
    ok, rows = True, []
    for mb in SHARD_MB:
        r = (mb << 20) // 512
        g = torch.Generator(device=run.dev).manual_seed(7 + run.rank)
        shard = torch.randn(r, 256, device=run.dev, generator=g).bfloat16()
        ref = torch.empty(run.world * r, 256, device=run.dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(ref, shard)
        y = op.run(shard)
        torch.cuda.synchronize()
        ok &= y is not None and run.ctx.find_block(y) is not None and torch.equal(y, ref)
        us = run.timed_us(lambda: op.run(shard))
        bus = (run.world - 1) * (mb << 20) / (us * 1e-6) / 1e9
        rows.append({"data_size": float(mb), "latency_avg": us, "throughput_avg": bus})
    run.finish(ok, rows)


if __name__ == "__main__":
    tasklib.guarded(main)
