"""In-place all-reduce of a bf16 tensor that lives in symmetric memory, reduced inside the
NVSwitch: one ``multimem.ld_reduce`` per 16-byte vector returns the sum over all ranks, one
``multimem.st`` writes it back to every rank.  Prints one JSON object.

Same exercise as the reference's datasets/example048_thunderkitten_all_reduce_easy (TK
``all_reduce`` over a parallel global layout, :64-94) and
datasets/example043_nccl_device_api_intranode_allreduce (``ncclMultimemReduceSumCopy``, :50-62).

Launched as: torchrun --nproc-per-node W ref_nvls_all_reduce.py
"""
import torch
import torch.distributed as dist

from commbench_b200.harness import tasklib
from commbench_b200.ops import collectives as coll

SIZES_MB = (1, 16, 64)


class NvlsAllReduce:
    """Owns one symmetric buffer of ``max_bytes``; ``run(n)`` all-reduces its first n elements."""

    def __init__(self, run: tasklib.TaskRun, max_bytes: int):
        self.ctx = run.ctx
        # --- solution: allocate the buffer in the symmetric heap (ctx.empty returns tensor, block)
        self.buf, _ = self.ctx.empty((max_bytes // 2,), torch.bfloat16)
        # --- end solution

    def run(self, n: int) -> torch.Tensor:
        """Sums the first n elements over all ranks, in place, through the multicast alias."""
        # --- solution: one launch of the in-switch all-reduce on the symmetric tensor
        #     (coll.all_reduce with algo="nvls"); return the reduced view
        return coll.all_reduce(self.ctx, self.buf[:n], algo="nvls")
        # --- end solution


def main():
    run = tasklib.start(min_world=2, heap_mb=256, need_multicast=True)
    op = NvlsAllReduce(run, max(SIZES_MB) << 20)
    ok, rows = True, []
    for mb in SIZES_MB:
        n = (mb << 20) // 2
        g = torch.Generator(device=run.dev).manual_seed(100 + run.rank)
        x = (torch.rand(n, device=run.dev, generator=g) * 2 - 1).bfloat16()
        ref = x.float()
        dist.all_reduce(ref)
        op.buf[:n].copy_(x)
        run.sync()
        y = op.run(n)
        torch.cuda.synchronize()
        ok &= y is not None and y.data_ptr() == op.buf.data_ptr()
        ok &= bool(((op.buf[:n].float() - ref).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))).item())
        us = run.timed_us(lambda: op.run(n))
        bus = 2.0 * (run.world - 1) / run.world * (mb << 20) / (us * 1e-6) / 1e9
        rows.append({"data_size": float(mb), "latency_avg": us, "throughput_avg": bus})
    run.finish(ok, rows)


if __name__ == "__main__":
    tasklib.guarded(main)
