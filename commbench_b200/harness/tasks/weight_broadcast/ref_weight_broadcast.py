"""Weight synchronisation from a trainer rank to inference ranks: a named state dict of many
tensors (mixed shapes and dtypes) is broadcast from rank 0, packed into a few flat buckets so
that the number of collective calls does not grow with the number of tensors.
Prints one JSON object.

Reference counterpart: datasets/example087_vllm_nccl_weight_transfer_engine (trainer -> inference
broadcast of a named state dict in buckets :127-176, sizes :398-410), here on CPU tensors with the
gloo backend so that it runs anywhere.

Launched as: torchrun --nproc-per-node W ref_weight_broadcast.py
"""
import json
import time

import torch
import torch.distributed as dist

TOTAL_MB = [1, 16, 64]
ITERS = 3
BUCKET_BYTES = 8 << 20


def make_state(total_bytes: int, seed: int) -> dict:
    """~total_bytes of parameters: 2-D weights, 1-D norms, a few odd shapes; fp32 / bf16 / fp16."""
    g = torch.Generator().manual_seed(seed)
    state, left, i = {}, total_bytes, 0
    dtypes = [torch.float32, torch.bfloat16, torch.float16]
    while left > 0:
        dt = dtypes[i % 3]
        esz = torch.empty(0, dtype=dt).element_size()
        rows = 64 + 32 * (i % 5)
        cols = max(8, min(left // (rows * esz), 1024 + 64 * (i % 7)))
        state[f"layers.{i}.weight"] = torch.randn(rows, cols, generator=g).to(dt)
        state[f"layers.{i}.norm"] = torch.randn(cols, generator=g).to(dt)
        left -= (rows * cols + cols) * esz
        i += 1
    state["step"] = torch.tensor(seed, dtype=torch.int64)
    state["empty"] = torch.empty(0, 3)
    return state


class WeightBroadcaster:
    def __init__(self):
        dist.init_process_group("gloo")
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.calls = 0

    def broadcast_state(self, state: dict, src: int = 0):
        """In place: after the call every rank's tensors hold rank `src`'s values.  Every rank
        passes a dict with the same keys, shapes and dtypes."""
        # --- solution: group the tensors by dtype in key order, pack consecutive tensors into flat
        #     buckets of at most BUCKET_BYTES (a tensor larger than that gets its own bucket),
        #     one dist.broadcast per bucket (count them in self.calls), copy back on the receivers;
        #     zero-element tensors need no traffic
        by_dtype: dict = {}
        for k, t in state.items():
            if t.numel():
                by_dtype.setdefault(t.dtype, []).append(t)
        for dt, tensors in by_dtype.items():
            bucket, size = [], 0
            for t in tensors + [None]:
                nbytes = 0 if t is None else t.numel() * t.element_size()
                if bucket and (t is None or size + nbytes > BUCKET_BYTES):
                    flat = torch.cat([b.reshape(-1) for b in bucket]) if self.rank == src else \
                        torch.empty(sum(b.numel() for b in bucket), dtype=dt)
                    dist.broadcast(flat, src=src)
                    self.calls += 1
                    if self.rank != src:
                        off = 0
                        for b in bucket:
                            b.copy_(flat[off:off + b.numel()].view_as(b))
                            off += b.numel()
                    bucket, size = [], 0
                if t is not None:
                    bucket.append(t)
                    size += nbytes
        # --- end solution

    def close(self):
        dist.destroy_process_group()


def same(a: dict, b: dict) -> bool:
    return list(a) == list(b) and all(
        a[k].dtype == b[k].dtype and a[k].shape == b[k].shape and
        torch.equal(a[k].reshape(-1).view(torch.uint8), b[k].reshape(-1).view(torch.uint8)) for k in a)


def main():
    wb = WeightBroadcaster()
    ok, rows = True, []
    for mb in TOTAL_MB:
        truth = make_state(mb << 20, seed=mb)                       # what rank 0 holds
        mine = truth if wb.rank == 0 else {k: torch.zeros_like(v) for k, v in truth.items()}
        before = wb.calls
        wb.broadcast_state(mine)
        calls = wb.calls - before
        ok &= same(mine, make_state(mb << 20, seed=mb))
        nbytes = sum(v.numel() * v.element_size() for v in truth.values())
        ok &= 1 <= calls <= nbytes // BUCKET_BYTES + 8               # buckets, not one call per tensor
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(ITERS):
            wb.broadcast_state(mine)
        dist.barrier()
        dt = (time.perf_counter() - t0) / ITERS
        rows.append({"data_size": nbytes / 2**20, "latency_avg": dt * 1e6, "throughput_avg": nbytes / dt / 1e9,
                     "tensors": len(truth), "calls": calls})
    flags = [None] * wb.world
    dist.all_gather_object(flags, bool(ok))
    if wb.rank == 0:
        print(json.dumps({"Correctness": "PASS" if all(flags) else "FAIL", "data_size_unit": "MB",
                          "latency_unit": "us", "throughput_unit": "GB/s", "metrics": rows}))
    wb.close()


if __name__ == "__main__":
    main()
