"""fp8 sequence-parallel column-parallel linear layer: C[M, N/W] = s_a * s_b *
(all_gather_rows(A_local) @ B_local^T) with e4m3 operands, one scale per tensor folded into the
epilogue, fp32 accumulation in tensor memory and the gather inside the GEMM kernel.
Prints one JSON object.

Same exercise as the reference's datasets/example052_thunderkitten_ag_gemm_fp8_easy (fp8 e4m3
tiles, :92-122) and datasets/example064_thunderkitten_ag_gemm_fp8_hard.

Launched as: torchrun --nproc-per-node W ref_ag_gemm_fp8_fused.py
"""
import torch
import torch.distributed as dist

from commbench_b200.harness import tasklib
from commbench_b200.ops.tp import AgGemm

M, N, K = 8192, 8192, 8192
F8 = torch.float8_e4m3fn


def quantize(x: torch.Tensor):
    """Per-tensor e4m3 quantisation: (values, scale) with x ~= values * scale."""
    scale = float(x.abs().max()) / 448.0
    return (x / scale).to(F8), scale


class Fp8AgGemm:
    def __init__(self, run: tasklib.TaskRun):
        self.ctx, self.W = run.ctx, run.world
        # TODO: the fused op, built for fp8 rows (dtype=torch.float8_e4m3fn)
        raise NotImplementedError

    def run(self, a_q, a_scale: float, b_q, b_scale: float) -> torch.Tensor:
        """a_q [M/W, K], b_q [N/W, K] e4m3 -> C [M, N/W] bf16 = a_scale * b_scale * (A @ B^T).
        Every rank quantised its rows with the SAME a_scale."""
        # TODO: one fused launch; the two scales go into alpha
        raise NotImplementedError


def main():
    run = tasklib.start(min_world=2, heap_mb=1024)
    W = run.world
    g = torch.Generator(device=run.dev).manual_seed(41 + run.rank)
    a = torch.randn(M // W, K, device=run.dev, generator=g) * 0.5
    b = torch.randn(N // W, K, device=run.dev, generator=g) * 0.05
    amax = a.abs().max()
    dist.all_reduce(amax, op=dist.ReduceOp.MAX)              # one activation scale for all ranks
    a_scale = float(amax) / 448.0
    a_q = (a / a_scale).to(F8)
    b_q, b_scale = quantize(b)
    op = Fp8AgGemm(run)
    c = op.run(a_q, a_scale, b_q, b_scale)
    torch.cuda.synchronize()
    # oracle: fp32 product of the same quantised values, sampled rows of the gathered A
    full_q = torch.empty(M, K, device=run.dev, dtype=torch.uint8)
    dist.all_gather_into_tensor(full_q, a_q.view(torch.uint8))
    rows = torch.arange(0, M, 61, device=run.dev)
    ref = (full_q.view(F8)[rows].float() @ b_q.float().t()) * (a_scale * b_scale)
    ok = c is not None and tuple(c.shape) == (M, N // W)
    ok = ok and bool(((c[rows].float() - ref).abs().max() <= 1.5e-2 * float(ref.abs().max())).item())
    us = run.timed_us(lambda: op.run(a_q, a_scale, b_q, b_scale))
    tflops = 2.0 * M * (N // W) * K / (us * 1e-6) / 1e12
    run.finish(ok, [{"data_size": M * K / 2**20, "latency_avg": us, "throughput_avg": tflops}],
               throughput_unit="TFLOP/s per rank")


if __name__ == "__main__":
    tasklib.guarded(main)
