"""Reduce-scatter: every rank holds W blocks; rank r must end up with the sum over ranks of
block r.  The backend at hand (gloo) has no reduce-scatter, so it has to be composed from what
there is, moving no more than an all-reduce would.  Checked against a reference that every rank
rebuilds locally from the seeds.  Prints one JSON object.

Launched as: torchrun --nproc-per-node W ref_reduce_scatter_blocks.py
"""
import json
import time

import torch
import torch.distributed as dist

BLOCK_ELEMS = [1 << 14, 1 << 18, 1 << 21]
ITERS = 3


class ReduceScatter:
    def __init__(self):
        dist.init_process_group("gloo")
        self.rank, self.world = dist.get_rank(), dist.get_world_size()

    def run(self, output: torch.Tensor, inp: torch.Tensor):
        """inp [W * n] (W blocks of n) on every rank; output [n] <- sum over ranks of block `rank`."""
        # TODO: one reduction per block with that block's owner as the root
        #       (dist.reduce, started asynchronously so that the W reductions overlap), then copy
        #       the own block out; an all_reduce of everything followed by a slice is also correct
        #       but every rank then receives W times what it needs
        raise NotImplementedError

    def close(self):
        dist.destroy_process_group()


def input_of(rank: int, world: int, n: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(7919 * rank + n)
    return torch.randint(-16, 17, (world * n,), generator=g).float()          # exact sums


def main():
    op = ReduceScatter()
    r, W = op.rank, op.world
    ok, rows = True, []
    for n in BLOCK_ELEMS:
        x = input_of(r, W, n)
        keep = x.clone()
        out = torch.empty(n)
        op.run(out, x)
        want = sum(input_of(q, W, n)[r * n:(r + 1) * n] for q in range(W))
        ok &= torch.equal(out, want) and torch.equal(x, keep)                 # the input is not clobbered
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(ITERS):
            op.run(out, x)
        dist.barrier()
        dt = (time.perf_counter() - t0) / ITERS
        nbytes = W * n * 4
        rows.append({"data_size": nbytes / 2**20, "latency_avg": dt * 1e6, "throughput_avg": nbytes / dt / 1e9})
    flags = [None] * W
    dist.all_gather_object(flags, bool(ok))
    if r == 0:
        print(json.dumps({"Correctness": "PASS" if all(flags) else "FAIL", "data_size_unit": "MB",
                          "latency_unit": "us", "throughput_unit": "GB/s", "metrics": rows}))
    op.close()


if __name__ == "__main__":
    main()
