"""Sequence-parallel <-> head-parallel re-sharding of a [B, N, H, D] activation with one
all-to-all each way (the Ulysses layouts).  Prints one JSON object.

Same exercise as the reference's datasets/example020_torch_distributed_nccl_alltoall (``Run(output, input, world,
scatter_idx, gather_idx)`` over ``all_to_all_single``, forward + inverse recovery check, :67-89),
on CPU tensors with the gloo backend so that it runs anywhere.

Launched as: torchrun --nproc-per-node W ref_ulysses_all_to_all.py
"""
import json
import time

import torch
import torch.distributed as dist

B, H, D = 1, 16, 64
SEQ = [1024, 4096, 16384]
ITERS = 5


class UlyssesAllToAll:
    def __init__(self):
        dist.init_process_group("gloo")
        self.rank, self.world = dist.get_rank(), dist.get_world_size()

    def to_heads(self, x: torch.Tensor) -> torch.Tensor:
        """[B, N/W, H, D] (this rank's sequence slice, all heads) -> [B, N, H/W, D]."""
        W = self.world
        b, n, h, d = x.shape
        send = x.reshape(b, n, W, h // W, d).permute(2, 0, 1, 3, 4).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send)
        return recv.permute(1, 0, 2, 3, 4).reshape(b, W * n, h // W, d)

    def to_sequence(self, x: torch.Tensor) -> torch.Tensor:
        """[B, N, H/W, D] (whole sequence, this rank's heads) -> [B, N/W, H, D]."""
        W = self.world
        b, n, h, d = x.shape
        send = x.reshape(b, W, n // W, h, d).permute(1, 0, 2, 3, 4).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send)
        return recv.permute(1, 2, 0, 3, 4).reshape(b, n // W, W * h, d)

    def close(self):
        dist.destroy_process_group()


def full_tensor(n: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(n)
    return torch.randn(B, n, H, D, generator=g)


def main():
    op = UlyssesAllToAll()
    r, W = op.rank, op.world
    ok, rows = True, []
    for n in SEQ:
        full = full_tensor(n)                                   # every rank can rebuild the whole tensor
        mine = full[:, r * n // W:(r + 1) * n // W].contiguous()
        heads = op.to_heads(mine)
        ok &= torch.equal(heads, full[:, :, r * H // W:(r + 1) * H // W])
        ok &= torch.equal(op.to_sequence(heads), mine)
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(ITERS):
            op.to_heads(mine)
        dist.barrier()
        dt = (time.perf_counter() - t0) / ITERS
        nbytes = mine.numel() * 4
        rows.append({"data_size": nbytes / 2**20, "latency_avg": dt * 1e6, "throughput_avg": nbytes / dt / 1e9})
    flags = [None] * W
    dist.all_gather_object(flags, bool(ok))
    if r == 0:
        print(json.dumps({"Correctness": "PASS" if all(flags) else "FAIL", "data_size_unit": "MB",
                          "latency_unit": "us", "throughput_unit": "GB/s", "metrics": rows}))
    op.close()


if __name__ == "__main__":
    main()
