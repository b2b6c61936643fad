"""Sequence-parallel column-parallel linear layer: C[M, N/W] = all_gather_rows(A_local) @ B_local^T
with the gather inside the GEMM kernel (communication CTAs push row blocks to the peers while
the tensor-core CTAs start on the rows that are already there).  Prints one JSON object.

Same exercise as the reference's datasets/example051_thunderkitten_ag_gemm_easy (comm / compute
CTA split at :118-150, CTA-pair main loop at :152-238).

Launched as: torchrun --nproc-per-node W ref_ag_gemm_fused.py
"""
import torch
import torch.distributed as dist

from commbench_b200.harness import tasklib
from commbench_b200.ops.tp import AgGemm

M, N, K = 8192, 8192, 8192          # global rows, global output columns, reduction


class FusedAgGemm:
    def __init__(self, run: tasklib.TaskRun):
        self.ctx, self.W = run.ctx, run.world
        # TODO: build the fused op once (it owns the gathered-A buffer and the row flags)
        raise NotImplementedError

    def run(self, a_local: torch.Tensor, b_local: torch.Tensor) -> torch.Tensor:
        """a_local [M/W, K], b_local [N/W, K] bf16 -> C [M, N/W] bf16, one kernel launch."""
        # TODO: call the fused op; no separate all-gather launch
        raise NotImplementedError


def main():
    run = tasklib.start(min_world=2, heap_mb=1024)
    W = run.world
    g = torch.Generator(device=run.dev).manual_seed(5 + run.rank)
    a = (torch.randn(M // W, K, device=run.dev, generator=g) * 0.5).bfloat16()
    b = (torch.randn(N // W, K, device=run.dev, generator=g) * 0.05).bfloat16()
    op = FusedAgGemm(run)
    c = op.run(a, b)
    torch.cuda.synchronize()
    full = torch.empty(M, K, device=run.dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(full, a)
    ref = full @ b.t()
    ok = c is not None and tuple(c.shape) == (M, N // W)
    ok = ok and bool(((c.float() - ref.float()).abs().max() <= 2e-2 * float(ref.float().abs().max())).item())
    us = run.timed_us(lambda: op.run(a, b))
    base = run.timed_us(lambda: torch.matmul(_ag(full, a), b.t()))
    tflops = 2.0 * M * (N // W) * K / (us * 1e-6) / 1e12
    rows = [{"data_size": M * K * 2 / 2**20, "latency_avg": us, "throughput_avg": tflops,
             "unfused_latency": base}]
    run.finish(ok, rows, throughput_unit="TFLOP/s per rank")


def _ag(full, a):
    dist.all_gather_into_tensor(full, a)
    return full


if __name__ == "__main__":
    tasklib.guarded(main)
