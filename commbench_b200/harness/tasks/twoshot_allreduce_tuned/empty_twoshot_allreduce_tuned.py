"""All-reduce without the switch: every rank sums its 1/W of the message over all ranks with
system-scope peer loads and stores each sum straight into every rank's symmetric buffer (the
push form of the two-shot algorithm: no second gather phase).  The candidate also picks the
launch shape - CTAs and 16-byte vectors in flight per thread - for each message size.
Prints one JSON object.

Same exercise as the reference's datasets/example031_msclpp_allreduce_rsag_zero_easy
(reduce-scatter + all-gather inside one kernel over peer pointers) and
datasets/example097_vllm_custom_all_reduce (size-dependent algorithm choice, :104-145).

Launched as: torchrun --nproc-per-node W ref_twoshot_allreduce_tuned.py
"""
import torch
import torch.distributed as dist

from commbench_b200.harness import tasklib
from commbench_b200.ops import collectives as coll

SIZES_MB = (1, 16, 64)


class PushAllReduce:
    def __init__(self, run: tasklib.TaskRun, max_bytes: int):
        self.ctx = run.ctx
        # TODO: the message lives in the symmetric heap
        raise NotImplementedError

    def launch_shape(self, nbytes: int) -> tuple[int, int]:
        """(CTAs, 16-byte vectors in flight per thread) for a message of nbytes."""
        # TODO: peer loads take ~2 us, so bytes in flight decide the rate: one CTA per
        #       64 KB of the per-rank share up to 128 CTAs, 8 vectors in flight from 4 MB up
        raise NotImplementedError

    def run(self, n: int) -> torch.Tensor:
        """In-place sum over ranks of the first n elements, plain peer loads/stores only."""
        # TODO: coll.all_reduce(..., algo="twoshot_push") with the chosen grid and unroll
        raise NotImplementedError


def main():
    run = tasklib.start(min_world=2, heap_mb=256)
    op = PushAllReduce(run, max(SIZES_MB) << 20)
    ok, rows = True, []
    for mb in SIZES_MB:
        n = (mb << 20) // 2
        g = torch.Generator(device=run.dev).manual_seed(200 + run.rank)
        x = (torch.rand(n, device=run.dev, generator=g) * 2 - 1).bfloat16()
        ref = x.float()
        dist.all_reduce(ref)
        op.buf[:n].copy_(x)
        run.sync()
        y = op.run(n)
        torch.cuda.synchronize()
        ok &= y is not None and y.data_ptr() == op.buf.data_ptr()
        ok &= bool(((op.buf[:n].float() - ref).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))).item())
        # every rank must hold the same bits (fixed summation order)
        mine = op.buf[:n].clone()
        other = mine.clone()
        dist.broadcast(other, src=0)
        ok &= torch.equal(mine, other)
        us = run.timed_us(lambda: op.run(n))
        nccl = x.clone()
        base = run.timed_us(lambda: dist.all_reduce(nccl))
        bus = 2.0 * (run.world - 1) / run.world * (mb << 20) / (us * 1e-6) / 1e9
        rows.append({"data_size": float(mb), "latency_avg": us, "throughput_avg": bus,
                     "nccl_latency": base})
    run.finish(ok, rows)


if __name__ == "__main__":
    tasklib.guarded(main)
