"""Pipeline-stage hand-off of a dictionary of tensors and plain values between two ranks:
metadata (keys, shapes, dtypes, non-tensor values) travels pickled, tensor payloads as
point-to-point messages.  Rank 1 echoes what it got; rank 0 checks byte equality.
Prints one JSON object.

Launched as: torchrun --nproc-per-node 2 empty_tensor_dict_handoff.py
"""
import json
import time

import torch
import torch.distributed as dist

ITERS = 5


class StageLink:
    def __init__(self):
        # TODO: initialise the process group (backend "gloo"); remember self.rank / self.world.
        raise NotImplementedError

    def send_tensor_dict(self, d: dict, dst: int):
        # TODO: send the metadata (key order, which entries are tensors, their shapes and dtypes,
        # the non-tensor values) as ONE pickled object, then every non-empty tensor with
        # dist.send, in key order.
        raise NotImplementedError

    def recv_tensor_dict(self, src: int) -> dict:
        # TODO: receive the metadata, allocate the tensors, receive the payloads; return a dict
        # with the same key order; zero-element tensors are rebuilt without a message.
        raise NotImplementedError

    def close(self):
        # TODO: tear the process group down.
        raise NotImplementedError


def make_dict(case: str) -> dict:
    g = torch.Generator().manual_seed(len(case))
    if case == "mixed":
        dtypes = [torch.float32, torch.float16, torch.bfloat16, torch.int64, torch.uint8, torch.bool]
        d = {f"t{i}": (torch.rand(3 + i, 5, generator=g) * 100).to(dtypes[i % len(dtypes)]) for i in range(50)}
        d.update({"step": 7, "name": "stage", "empty": torch.empty(0, 4), "flags": [1, 2, 3]})
        return d
    nbytes = {"16KiB": 16 << 10, "1MiB": 1 << 20, "16MiB": 16 << 20}[case]
    return {"hidden": torch.rand(nbytes // 4, generator=g), "step": 1}


def same(a: dict, b: dict) -> bool:
    if list(a) != list(b):
        return False
    for k in a:
        if isinstance(a[k], torch.Tensor):
            if not (isinstance(b[k], torch.Tensor) and a[k].dtype == b[k].dtype and a[k].shape == b[k].shape
                    and torch.equal(a[k].view(torch.uint8) if a[k].numel() else a[k],
                                    b[k].view(torch.uint8) if b[k].numel() else b[k])):
                return False
        elif a[k] != b[k]:
            return False
    return True


def main():
    link = StageLink()
    ok, rows = True, []
    for case in ("16KiB", "1MiB", "16MiB", "mixed"):
        d = make_dict(case)
        nbytes = sum(v.numel() * v.element_size() for v in d.values() if isinstance(v, torch.Tensor))
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(ITERS):
            if link.rank == 0:
                link.send_tensor_dict(d, 1)
                ok &= same(d, link.recv_tensor_dict(1))
            elif link.rank == 1:
                link.send_tensor_dict(link.recv_tensor_dict(0), 0)
        dt = (time.perf_counter() - t0) / ITERS
        rows.append({"data_size": nbytes / 2**20, "latency_avg": dt * 1e6, "throughput_avg": 2 * nbytes / dt / 1e9})
    if link.rank == 0:
        print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "MB", "latency_unit": "us",
                          "throughput_unit": "GB/s", "metrics": rows}))
    link.close()


if __name__ == "__main__":
    main()
