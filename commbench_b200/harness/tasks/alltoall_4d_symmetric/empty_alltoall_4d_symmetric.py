"""Sequence-parallel <-> head-parallel re-sharding of a [B, S/W, H, D] bf16 activation on the
GPUs, one kernel launch each way, reading the peers' symmetric tensors directly (no pack /
unpack passes around a flat all-to-all).  Prints one JSON object.

Same exercise as the reference's datasets/example049_thunderkitten_alltoall_easy (4-D TMA
all-to-all with scatter / gather axes, :60-121) and the device half of
datasets/example020_torch_distributed_nccl_alltoall (:67-89).

Launched as: torchrun --nproc-per-node W ref_alltoall_4d_symmetric.py
"""
import torch
import torch.distributed as dist

from commbench_b200.harness import tasklib
from commbench_b200.ops import collectives as coll

B, H, D = 1, 32, 128
SEQ_LOCAL = (1024, 4096, 16384)


class UlyssesExchange:
    def __init__(self, run: tasklib.TaskRun):
        self.ctx, self.W = run.ctx, run.world
        s = max(SEQ_LOCAL)
        # TODO: both inputs live in the symmetric heap so that peers can read them
        raise NotImplementedError

    def to_heads(self, s_local: int) -> torch.Tensor:
        """self.seq_sharded[:, :s_local] ([B, S/W, H, D]) -> [B, S, H/W, D] (ordinary tensor)."""
        # TODO: coll.all_to_all_4d(..., to_heads=True) on a contiguous symmetric view
        raise NotImplementedError

    def to_sequence(self, s_local: int) -> torch.Tensor:
        """self.head_sharded ([B, S, H/W, D]) -> [B, S/W, H, D] (ordinary tensor)."""
        # TODO: the inverse exchange, to_heads=False
        raise NotImplementedError


def main():
    run = tasklib.start(min_world=2, heap_mb=1024)
    W, r = run.world, run.rank
    op = UlyssesExchange(run)
    ok, rows = True, []
    for s in SEQ_LOCAL:
        g = torch.Generator(device=run.dev).manual_seed(s)          # same full tensor on every rank
        full = torch.randn(B, s * W, H, D, device=run.dev, generator=g).bfloat16()
        mine = full[:, r * s:(r + 1) * s].contiguous()
        op.seq_sharded.view(-1)[: mine.numel()].copy_(mine.view(-1))
        run.sync()
        heads = op.to_heads(s)
        torch.cuda.synchronize()
        ok &= heads is not None and torch.equal(heads, full[:, :, r * H // W:(r + 1) * H // W])
        op.head_sharded.view(-1)[: heads.numel()].copy_(heads.reshape(-1))
        run.sync()
        back = op.to_sequence(s)
        torch.cuda.synchronize()
        ok &= back is not None and torch.equal(back, mine)
        us = run.timed_us(lambda: op.to_heads(s))
        nbytes = mine.numel() * 2
        rows.append({"data_size": nbytes / 2**20, "latency_avg": us,
                     "throughput_avg": (W - 1) / W * nbytes / (us * 1e-6) / 1e9})
    run.finish(ok, rows)


if __name__ == "__main__":
    tasklib.guarded(main)
