"""Causal attention over a sequence sharded across GPUs (Ulysses form): rank r attends for its
slice of the heads over the WHOLE sequence, and both re-shardings happen inside the attention
kernel - key / value head slices are pulled from the peers, query tiles are loaded from their
owners' memory, output rows are stored to their owners.  Prints one JSON object.

Same exercise as the reference's datasets/example058_thunderkitten_ulysses_attn_easy (4-D
exchange at :59-120, attention between the two exchanges at :330-359).

Launched as: torchrun --nproc-per-node W ref_ulysses_attention_kernel.py
"""
import torch

from commbench_b200.harness import tasklib
from commbench_b200.ops.cp import UlyssesAttention

B, HQ, HKV, D = 1, 16, 4, 128
S_LOCAL = 4096


class UlyssesCausalAttention:
    def __init__(self, run: tasklib.TaskRun):
        self.ctx = run.ctx
        # --- solution: build the op once; its q/k/v/o buffers live in symmetric memory
        self.op = UlyssesAttention(self.ctx, B, S_LOCAL, HQ, HKV)
        # --- end solution

    def run(self, q, k, v) -> torch.Tensor:
        """q [B, S/W, HQ, D], k / v [B, S/W, HKV, D] bf16 (this rank's contiguous sequence
        slice, all heads) -> o [B, S/W, HQ, D]."""
        # --- solution: one forward (inputs are copied into the symmetric buffers); returns o_buf
        return self.op.forward(q, k, v, causal=True)
        # --- end solution


def main():
    run = tasklib.start(min_world=2, heap_mb=1024)
    W, r = run.world, run.rank
    S = S_LOCAL * W
    op = UlyssesCausalAttention(run)
    g = torch.Generator(device=run.dev).manual_seed(29)
    qf = torch.randn(B, S, HQ, D, device=run.dev, generator=g).bfloat16()
    kf = torch.randn(B, S, HKV, D, device=run.dev, generator=g).bfloat16()
    vf = torch.randn(B, S, HKV, D, device=run.dev, generator=g).bfloat16()
    sl = slice(r * S_LOCAL, (r + 1) * S_LOCAL)
    q, k, v = (t[:, sl].contiguous() for t in (qf, kf, vf))
    o = op.run(q, k, v)
    torch.cuda.synchronize()
    ok = o is not None and tuple(o.shape) == (B, S_LOCAL, HQ, D)
    for h in (0, HQ - 1):
        kv = h // (HQ // HKV)
        s = (qf[0, sl, h].float() @ kf[0, :, kv].float().t()) / D ** 0.5
        rows = torch.arange(r * S_LOCAL, (r + 1) * S_LOCAL, device=run.dev)[:, None]
        s.masked_fill_(torch.arange(S, device=run.dev)[None, :] > rows, float("-inf"))
        ref = torch.softmax(s, -1) @ vf[0, :, kv].float()
        ok = ok and bool(((o[0, :, h].float() - ref).abs().max() < 2e-2).item())
    us = run.timed_us(lambda: op.run(q, k, v), iters=5, warmup=2)
    flops = 4.0 * B * HQ * S * S * D / 2 / W
    run.finish(ok, [{"data_size": q.numel() * 2 / 2**20, "latency_avg": us,
                     "throughput_avg": flops / (us * 1e-6) / 1e12}],
               throughput_unit="TFLOP/s per rank")


if __name__ == "__main__":
    tasklib.guarded(main)
