"""Expert-parallel MoE feed-forward: route every token to its top-k experts on other GPUs
(fp8 payload + per-128 scales over NVLink), run the grouped up / SwiGLU / down GEMMs on the
rows that arrived, send the results back and combine them with the routing weights.
Prints one JSON object.

Same exercise as the reference's datasets/example056_thunderkitten_moe_dispatch_gemm_easy
(dispatch with per-row-block arrival counters at :181-202, grouped GEMM at :266-293) and the
DeepEP layout / dispatch / combine family (datasets/example042_deepep_dispatch_layout,
datasets/example047_deepep_intranode_notify_dispatch).

Launched as: torchrun --nproc-per-node W ref_moe_dispatch_gemm.py
"""
import torch

from commbench_b200.harness import tasklib
from commbench_b200.ops.moe import MoELayer, reference_moe, router_topk

T, H, I, E, K = 1024, 2048, 1024, 32, 4      # tokens per rank, hidden, intermediate, experts, top-k


class ExpertParallelFfn:
    def __init__(self, run: tasklib.TaskRun):
        self.ctx = run.ctx
        # --- solution: build the layer once: it owns the receive buffers, counters and the
        #     (random) expert weights of this rank
        self.layer = MoELayer(self.ctx, T, H, I, E, K, capacity_factor=2.0, seed=3)
        # --- end solution

    def weights(self):
        """(w1 [E/W, 2I, H], w2 [E/W, H, I]) of the experts this rank hosts."""
        # --- solution: the layer's own weights
        return self.layer.weights()
        # --- end solution

    def run(self, x, topk_idx, topk_w) -> torch.Tensor:
        """x [T, H] bf16, topk_idx [T, K] int32, topk_w [T, K] fp32 -> y [T, H] bf16."""
        # --- solution: one forward of the layer (dispatch, grouped GEMMs, combine)
        return self.layer.forward(x, topk_idx, topk_w)
        # --- end solution


def main():
    import torch.distributed as dist

    run = tasklib.start(min_world=2, heap_mb=2048)
    W = run.world
    op = ExpertParallelFfn(run)
    g = torch.Generator(device=run.dev).manual_seed(17 + run.rank)
    x = torch.randn(T, H, device=run.dev, generator=g).bfloat16()
    idx, w = router_topk(torch.randn(T, E, device=run.dev, generator=g), K)
    y = op.run(x, idx, w)
    torch.cuda.synchronize()
    # oracle: every rank gathers all expert weights and evaluates its own tokens densely in fp32
    w1, w2 = op.weights()
    w1_all = torch.empty((W,) + tuple(w1.shape), device=run.dev, dtype=w1.dtype)
    w2_all = torch.empty((W,) + tuple(w2.shape), device=run.dev, dtype=w2.dtype)
    dist.all_gather_into_tensor(w1_all, w1.contiguous())
    dist.all_gather_into_tensor(w2_all, w2.contiguous())
    ref = reference_moe(x, idx, w, w1_all.flatten(0, 1), w2_all.flatten(0, 1), I)
    err = float(((y.float() - ref.float()).abs().max() / (ref.float().abs().max() + 1e-9)).item())
    ok = y is not None and tuple(y.shape) == (T, H) and err < 6e-2
    us = run.timed_us(lambda: op.run(x, idx, w))
    tflops = 2.0 * T * K * H * 3 * I / (us * 1e-6) / 1e12
    run.finish(ok, [{"data_size": T * H * 2 / 2**20, "latency_avg": us, "throughput_avg": tflops}],
               max_rel_err=err, throughput_unit="TFLOP/s per rank")


if __name__ == "__main__":
    tasklib.guarded(main)
