"""All-reduce over torch.distributed (gloo, CPU).  Prints one JSON object.

Launched as: torchrun --nproc-per-node W ref_gloo_allreduce.py
"""
import json
import time

import torch
import torch.distributed as dist

NUMEL = 1 << 20
ITERS = 5


class AllReduce:
    def __init__(self):
        dist.init_process_group("gloo")
        self.rank, self.world = dist.get_rank(), dist.get_world_size()

    def make_input(self, rank: int) -> torch.Tensor:
        g = torch.Generator().manual_seed(rank)
        return torch.rand(NUMEL, generator=g, dtype=torch.float32)

    def run(self, x: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(x)
        return x

    def reference(self) -> torch.Tensor:
        return sum(self.make_input(r).double() for r in range(self.world))

    def close(self):
        dist.destroy_process_group()


def main():
    ar = AllReduce()
    x = ar.make_input(ar.rank)
    out = ar.run(x.clone())
    ok = torch.allclose(out.double(), ar.reference(), rtol=1e-5, atol=1e-6)
    t0 = time.perf_counter()
    for _ in range(ITERS):
        ar.run(x.clone())
    dt = (time.perf_counter() - t0) / ITERS
    if ar.rank == 0:
        nbytes = NUMEL * 4
        print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "MB",
                          "latency_unit": "us", "throughput_unit": "GB/s",
                          "metrics": [{"data_size": nbytes / 2**20, "latency_avg": dt * 1e6,
                                       "throughput_avg": nbytes / dt / 1e9}]}))
    ar.close()


if __name__ == "__main__":
    main()
