"""All-reduce over torch.distributed (gloo, CPU).  Prints one JSON object.

Launched as: torchrun --nproc-per-node W empty_gloo_allreduce.py
"""
import json
import time

import torch
import torch.distributed as dist

NUMEL = 1 << 20
ITERS = 5


class AllReduce:
    def __init__(self):
        # TODO: initialise the process group (backend "gloo") and remember rank / world size.
        raise NotImplementedError

    def make_input(self, rank: int) -> torch.Tensor:
        # TODO: float32 tensor of NUMEL elements from torch.manual_seed(rank), uniform in [0, 1).
        raise NotImplementedError

    def run(self, x: torch.Tensor) -> torch.Tensor:
        # TODO: sum over all ranks, in place, and return the tensor.
        raise NotImplementedError

    def reference(self) -> torch.Tensor:
        # TODO: float64 sum of every rank's input, recomputed locally from the seeds.
        raise NotImplementedError

    def close(self):
        # TODO: tear the process group down.
        raise NotImplementedError


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
