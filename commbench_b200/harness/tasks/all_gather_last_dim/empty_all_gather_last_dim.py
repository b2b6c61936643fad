"""All-gather along the LAST dimension: every rank holds a column slice [rows, cols / W] of a
matrix and must end up with the whole [rows, cols] matrix - the collective gathers along dim 0,
so the result has to be put back in column order without an extra pass per rank where possible.
Prints one JSON object.

Launched as: torchrun --nproc-per-node W ref_all_gather_last_dim.py
"""
import json
import time

import torch
import torch.distributed as dist

ROWS = 256
COLS = [1024, 4096, 16384]
ITERS = 5


class AllGather:
    def __init__(self):
        dist.init_process_group("gloo")
        self.rank, self.world = dist.get_rank(), dist.get_world_size()

    def all_gather_last_dim(self, x: torch.Tensor) -> torch.Tensor:
        """x [..., c] on every rank -> [..., W * c], rank r's slice at columns r*c .. (r+1)*c."""
        # TODO: one collective: gather the slices as W blocks along a new leading
        #       dimension, then move that dimension next to the last one and merge them
        #       (movedim + reshape; one copy)
        raise NotImplementedError

    def close(self):
        dist.destroy_process_group()


def full_matrix(cols: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(cols)
    return torch.randn(ROWS, cols, generator=g)


def main():
    op = AllGather()
    r, W = op.rank, op.world
    ok, rows = True, []
    for cols in COLS:
        full = full_matrix(cols)
        c = cols // W
        mine = full[:, r * c:(r + 1) * c]                      # a non-contiguous view on purpose
        out = op.all_gather_last_dim(mine)
        ok &= out.shape == full.shape and torch.equal(out, full)
        batched = op.all_gather_last_dim(mine.reshape(4, ROWS // 4, c))      # leading dims are kept
        ok &= torch.equal(batched, full.reshape(4, ROWS // 4, cols))
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(ITERS):
            op.all_gather_last_dim(mine)
        dist.barrier()
        dt = (time.perf_counter() - t0) / ITERS
        nbytes = full.numel() * 4
        rows.append({"data_size": nbytes / 2**20, "latency_avg": dt * 1e6, "throughput_avg": nbytes / dt / 1e9})
    flags = [None] * W
    dist.all_gather_object(flags, bool(ok))
    if r == 0:
        print(json.dumps({"Correctness": "PASS" if all(flags) else "FAIL", "data_size_unit": "MB",
                          "latency_unit": "us", "throughput_unit": "GB/s", "metrics": rows}))
    op.close()


if __name__ == "__main__":
    main()
