"""Causal attention over a sequence sharded across GPUs (context parallelism, ring form): every
rank keeps its queries, pulls the key / value shards of the other ranks while it attends to the
shards it already has, and carries the running softmax state across all shards - one kernel
launch per call, zig-zag sharding so that causal work is balanced.  Prints one JSON object.

Same exercise as the reference's datasets/example057_thunderkitten_ring_attn_easy (7+7 warp
KV ring with double-buffered K/V at :97-134, stage schedule at :336-379).

Launched as: torchrun --nproc-per-node W ref_ring_attention_kernel.py
"""
import torch

from commbench_b200.harness import tasklib
from commbench_b200.ops.cp import RingAttention, zigzag_shard

B, HQ, HKV, D = 1, 16, 4, 128
S_LOCAL = 4096


class RingCausalAttention:
    def __init__(self, run: tasklib.TaskRun):
        self.ctx = run.ctx
        # TODO: build the op once; zig-zag sharding (rank r holds chunks r and 2W-1-r)
        raise NotImplementedError

    def shard(self, full: torch.Tensor) -> torch.Tensor:
        """This rank's rows of a full-sequence tensor [B, S, heads, D] under the op's sharding."""
        # TODO: zigzag_shard(full, world, rank)
        raise NotImplementedError

    def run(self, q, k, v) -> torch.Tensor:
        """q [B, S/W, HQ, D], k / v [B, S/W, HKV, D] bf16 -> o [B, S/W, HQ, D]."""
        # TODO: one forward; returns (o, lse)
        raise NotImplementedError


def main():
    run = tasklib.start(min_world=2, heap_mb=1024)
    W = run.world
    S = S_LOCAL * W
    op = RingCausalAttention(run)
    g = torch.Generator(device=run.dev).manual_seed(23)              # same full tensors on every rank
    qf = torch.randn(B, S, HQ, D, device=run.dev, generator=g).bfloat16()
    kf = torch.randn(B, S, HKV, D, device=run.dev, generator=g).bfloat16()
    vf = torch.randn(B, S, HKV, D, device=run.dev, generator=g).bfloat16()
    q, k, v = (op.shard(t).contiguous() for t in (qf, kf, vf))
    o = op.run(q, k, v)
    torch.cuda.synchronize()
    # oracle: full-sequence attention in fp32 for a sample of heads, sharded the same way
    ok = o is not None and tuple(o.shape) == (B, S_LOCAL, HQ, D)
    for h in (0, HQ - 1):
        kv = h // (HQ // HKV)
        s = (qf[0, :, h].float() @ kf[0, :, kv].float().t()) / D ** 0.5
        s.masked_fill_(torch.ones(S, S, device=run.dev, dtype=torch.bool).triu(1), float("-inf"))
        ref = (torch.softmax(s, -1) @ vf[0, :, kv].float())[None, :, None, :]
        ref_local = op.shard(ref)[0, :, 0]
        ok = ok and bool(((o[0, :, h].float() - ref_local).abs().max() < 2e-2).item())
    us = run.timed_us(lambda: op.run(q, k, v), iters=5, warmup=2)
    flops = 4.0 * B * HQ * S * S * D / 2 / W                          # causal, per rank
    run.finish(ok, [{"data_size": q.numel() * 2 / 2**20, "latency_avg": us,
                     "throughput_avg": flops / (us * 1e-6) / 1e12}],
               throughput_unit="TFLOP/s per rank")


if __name__ == "__main__":
    tasklib.guarded(main)
