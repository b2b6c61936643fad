"""Row-parallel linear layer with a replicated output: out[M, N] = all_reduce(A[M, K/W] @
B[N, K/W]^T) in one kernel: the owner of an output tile adds the W partial tiles in fp32 as
they arrive and stores the sum to every rank.  Prints one JSON object.

Same exercise as the reference's datasets/example053_thunderkitten_gemm_ar_easy (GEMM, barrier,
multimem all-reduce, barrier as separate launches at :200-238 and :528-536; here they are one).

Launched as: torchrun --nproc-per-node W ref_gemm_ar_fused.py
"""
import torch
import torch.distributed as dist

from commbench_b200.harness import tasklib
from commbench_b200.ops.tp import GemmAr

N, K = 8192, 8192
ROWS = (128, 1024, 4096)


class FusedGemmAr:
    def __init__(self, run: tasklib.TaskRun):
        self.ctx, self.W = run.ctx, run.world
        # TODO: build the fused op once for the largest M
        raise NotImplementedError

    def run(self, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """a [M, K/W], b [N, K/W] bf16 -> out [M, N] = sum over ranks, on every rank."""
        # TODO: call the fused op with the caller's output tensor
        raise NotImplementedError


def main():
    run = tasklib.start(min_world=2, heap_mb=1024)
    W = run.world
    op = FusedGemmAr(run)
    g = torch.Generator(device=run.dev).manual_seed(13 + run.rank)
    b = (torch.randn(N, K // W, device=run.dev, generator=g) * 0.05).bfloat16()
    ok, rows = True, []
    for m in ROWS:
        a = (torch.randn(m, K // W, device=run.dev, generator=g) * 0.5).bfloat16()
        out = torch.empty(m, N, device=run.dev, dtype=torch.bfloat16)
        y = op.run(a, b, out)
        torch.cuda.synchronize()
        ref = (a @ b.t()).float()
        dist.all_reduce(ref)
        ok &= y is not None and bool(((out.float() - ref).abs().max() <= 2e-2 * float(ref.abs().max())).item())
        us = run.timed_us(lambda: op.run(a, b, out))
        tmp = torch.empty(m, N, device=run.dev, dtype=torch.bfloat16)
        base = run.timed_us(lambda: dist.all_reduce(torch.matmul(a, b.t(), out=tmp)))
        rows.append({"data_size": m * N * 2 / 2**20, "latency_avg": us,
                     "throughput_avg": 2.0 * m * N * (K // W) / (us * 1e-6) / 1e12,
                     "unfused_latency": base})
    run.finish(ok, rows, throughput_unit="TFLOP/s per rank")


if __name__ == "__main__":
    tasklib.guarded(main)
