"""Device-side barrier across GPUs, two designs timed back to back: the flag matrix (every rank
stores one word to every peer and waits for W words) and the multicast counter (one
``multimem.red`` bumps a counter on every rank).  Prints one JSON object.

Same exercise as the reference's datasets/example017_intranode_gpu_barrier (add/sub matrix
barrier, latency loop at :114-125) and the multimem barrier of
datasets/example048_thunderkitten_all_reduce_easy (:96-115).

Launched as: torchrun --nproc-per-node W ref_nvls_barrier_latency.py
"""
import torch

from commbench_b200.harness import tasklib
from commbench_b200.ops import collectives as coll

ITERS = 200


class DeviceBarrier:
    def __init__(self, run: tasklib.TaskRun):
        self.ctx = run.ctx

    def run(self, iters: int, use_nvls: bool):
        """`iters` barriers back to back inside ONE launch."""
        # TODO: coll.barrier runs the loop on the device (one <<<1,32>>> launch);
        #       use_nvls picks the multimem.red counter instead of the flag matrix
        raise NotImplementedError


def main():
    run = tasklib.start(min_world=2, heap_mb=64, need_multicast=True)
    op = DeviceBarrier(run)
    ok, rows = True, []
    for i, use_nvls in enumerate((False, True)):
        # a rank that is late on the host must hold the others back: the barrier really waits
        if run.rank == 0:
            torch.cuda._sleep(20_000_000)
        op.run(1, use_nvls)
        torch.cuda.synchronize()
        base = run.timed_us(lambda: op.run(1, use_nvls), iters=5, warmup=2)
        loop = run.timed_us(lambda: op.run(ITERS, use_nvls), iters=5, warmup=2)
        per = max(loop - base, 0.0) / (ITERS - 1)
        ok &= 0.0 < per < 100.0
        rows.append({"data_size": float(i), "latency_avg": per, "throughput_avg": 1.0 / max(per, 1e-9)})
    try:
        run.ctx.check_status(sync=True)
    except Exception:
        ok = False
    run.finish(ok, rows)


if __name__ == "__main__":
    tasklib.guarded(main)
