"""Sequence-parallel <-> head-parallel re-sharding of a [B, N, H, D] activation with one
all-to-all each way (the Ulysses layouts).  Prints one JSON object.

Launched as: torchrun --nproc-per-node W empty_ulysses_all_to_all.py
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
        # TODO: initialise the process group (backend "gloo"); remember self.rank / self.world.
        raise NotImplementedError

    def to_heads(self, x: torch.Tensor) -> torch.Tensor:
        """[B, N/W, H, D] (this rank's sequence slice, all heads) -> [B, N, H/W, D]."""
        # TODO: one dist.all_to_all_single; rank r ends up with heads r*H/W ... (r+1)*H/W of the
        # whole sequence, sequence positions in global order.
        raise NotImplementedError

    def to_sequence(self, x: torch.Tensor) -> torch.Tensor:
        """[B, N, H/W, D] (whole sequence, this rank's heads) -> [B, N/W, H, D]."""
        # TODO: the inverse of to_heads, again one all_to_all_single.
        raise NotImplementedError

    def close(self):
        # TODO: tear the process group down.
        raise NotImplementedError


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
