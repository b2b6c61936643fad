"""Row-parallel linear layer with a sequence-parallel output: out[M/W, N] =
reduce_scatter_rows(A[M, K/W] @ B[N, K/W]^T), the reduction running inside the GEMM kernel (each
partial tile goes to the rank that owns its rows as soon as it leaves the tensor cores).
Prints one JSON object.

Same exercise as the reference's datasets/example054_thunderkitten_gemm_rs_easy (task rotation
and in-flight reduce at :112-139, :141-208).

Launched as: torchrun --nproc-per-node W ref_gemm_rs_fused.py
"""
import torch
import torch.distributed as dist

from commbench_b200.harness import tasklib
from commbench_b200.ops.tp import GemmRs

M, N, K = 8192, 8192, 8192          # global rows, output columns, global reduction


class FusedGemmRs:
    def __init__(self, run: tasklib.TaskRun):
        self.ctx, self.W = run.ctx, run.world
        # TODO: build the fused op once (it owns the staging slots and the tile flags)
        raise NotImplementedError

    def run(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        """a [M, K/W], b [N, K/W] bf16 -> this rank's rows of the sum over ranks, [M/W, N]."""
        # TODO: call the fused op; no separate reduce-scatter launch
        raise NotImplementedError


def main():
    run = tasklib.start(min_world=2, heap_mb=1024)
    W = run.world
    g = torch.Generator(device=run.dev).manual_seed(9 + run.rank)
    a = (torch.randn(M, K // W, device=run.dev, generator=g) * 0.5).bfloat16()
    b = (torch.randn(N, K // W, device=run.dev, generator=g) * 0.05).bfloat16()
    op = FusedGemmRs(run)
    y = op.run(a, b)
    torch.cuda.synchronize()
    part = (a @ b.t()).float()
    ref = torch.empty(M // W, N, device=run.dev, dtype=torch.float32)
    dist.reduce_scatter_tensor(ref, part)
    ok = y is not None and tuple(y.shape) == (M // W, N)
    ok = ok and bool(((y.float() - ref).abs().max() <= 2e-2 * float(ref.abs().max())).item())
    us = run.timed_us(lambda: op.run(a, b))
    out = torch.empty(M // W, N, device=run.dev, dtype=torch.bfloat16)
    base = run.timed_us(lambda: dist.reduce_scatter_tensor(out, a @ b.t()))
    tflops = 2.0 * M * N * (K // W) / (us * 1e-6) / 1e12
    rows = [{"data_size": M * N * 2 / 2**20, "latency_avg": us, "throughput_avg": tflops,
             "unfused_latency": base}]
    run.finish(ok, rows, throughput_unit="TFLOP/s per rank")


if __name__ == "__main__":
    tasklib.guarded(main)
