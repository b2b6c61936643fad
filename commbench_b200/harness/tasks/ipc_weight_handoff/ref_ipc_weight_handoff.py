"""Weight hand-off between two processes on ONE GPU without a host copy: a trainer process exports
a weight tensor as a CUDA-IPC handle, an inference process maps the same allocation and copies it
into its own weights (device to device).  Prints one JSON object.

Reference counterpart: datasets/example088_vllm_ipc_weight_transfer_engine (``reduce_tensor``
style handle export, rebuild in the worker, ``load_weights``).

Run as: python ref_ipc_weight_handoff.py
"""
import json
import time

import torch

ROWS, COLS = 2048, 2048


def consumer(handle, q):
    """Runs in the second process: map, copy into local weights, report (shape, checksum, seconds)."""
    import torch as t

    from commbench_b200.ops.util import ipc_import

    # --- solution: w = ipc_import(handle) maps the producer's memory (no copy); allocate local
    #     weights, time local.copy_(w) with a synchronize on both sides, put
    #     (tuple(w.shape), float(local.double().sum()), seconds) on the queue
    w = ipc_import(handle)
    local = t.empty_like(w)
    t.cuda.synchronize()
    t0 = time.perf_counter()
    local.copy_(w)
    t.cuda.synchronize()
    dt = time.perf_counter() - t0
    q.put((tuple(w.shape), float(local.double().sum().item()), dt))
    # --- end solution


class WeightHandoff:
    def send(self, w: torch.Tensor):
        """Starts the consumer process with an IPC handle of `w`; returns its report."""
        import torch.multiprocessing as mp

        from commbench_b200.ops.util import ipc_export

        # --- solution: spawn context, Queue, Process(target=consumer, args=(ipc_export(w), q));
        #     wait for the report with a time-out, join, check the exit code
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        p = ctx.Process(target=consumer, args=(ipc_export(w), q))
        p.start()
        report = q.get(timeout=240)
        p.join(60)
        if p.exitcode != 0:
            raise RuntimeError(f"consumer exited with {p.exitcode}")
        return report
        # --- end solution


def main():
    if not torch.cuda.is_available():
        print(json.dumps({"Correctness": "SKIP", "reason": "no CUDA device", "metrics": []}))
        return
    w = torch.arange(ROWS * COLS, device="cuda", dtype=torch.float32).view(ROWS, COLS) % 1021
    expect = float(w.double().sum().item())
    shape, total, dt = WeightHandoff().send(w)
    ok = shape == (ROWS, COLS) and total == expect and dt > 0
    nbytes = ROWS * COLS * 4
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "MB", "latency_unit": "us",
                      "throughput_unit": "GB/s",
                      "metrics": [{"data_size": nbytes / 2**20, "latency_avg": dt * 1e6,
                                   "throughput_avg": nbytes / dt / 1e9}]}))


if __name__ == "__main__":
    main()
