"""Tiled producer / consumer hand-off through memory a peer can write: the producer copies a
matrix tile by tile into the consumer's buffer and raises one flag per tile; the consumer waits
(bounded) for each tile's flag and reduces the tile as soon as it is there.  Prints one JSON
object.

Reference counterpart: datasets/example035_nvshmem_tiled_produce_consume (``nvshmemx_putmem_signal``
per tile, ``nvshmem_signal_wait_until`` in the consumer), on this package's one-sided primitives
(``ops.shmem.tile_put`` / ``tile_consume``); on one GPU the "peer" buffer is a local tensor.

Run as: python ref_tile_produce_consume.py
"""
import json

import torch

TILE = 64
SIDES = (256, 1024, 4096)


class TiledHandoff:
    def run(self, src: torch.Tensor, remote: torch.Tensor, flags: torch.Tensor, value: int):
        """Producer: src -> remote in TILE x TILE tiles, flag[t] = value after tile t.  Consumer:
        per-tile sums of `remote`, each taken after its flag.  Returns (sums, device status)."""
        from commbench_b200.ops import shmem

        # --- solution: shmem.tile_put(remote.data_ptr(), src, TILE, flags.data_ptr(), value=value),
        #     then shmem.tile_consume(remote, TILE, flags.data_ptr(), value=value, status=st)
        st = torch.zeros(1, dtype=torch.int32, device="cuda")
        shmem.tile_put(remote.data_ptr(), src, TILE, flags.data_ptr(), value=value)
        part = shmem.tile_consume(remote, TILE, flags.data_ptr(), value=value, status=st)
        return part, st
        # --- end solution


def main():
    if not torch.cuda.is_available():
        print(json.dumps({"Correctness": "SKIP", "reason": "no CUDA device", "metrics": []}))
        return
    h = TiledHandoff()
    ok, rows = True, []
    for side in SIDES:
        g = torch.Generator(device="cuda").manual_seed(side)
        src = torch.randn(side, side, device="cuda", generator=g)
        remote = torch.zeros_like(src)
        flags = torch.zeros((side // TILE) ** 2, dtype=torch.int32, device="cuda")
        part, st = h.run(src, remote, flags, 1)
        torch.cuda.synchronize()
        ref = src.view(side // TILE, TILE, side // TILE, TILE).sum(dim=(1, 3)).reshape(-1)
        ok &= part is not None and int(st.item()) == 0 and torch.equal(remote, src)
        ok &= torch.allclose(part, ref, atol=1e-2, rtol=1e-4)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for it in range(10):
            h.run(src, remote, flags, 2 + it)           # flags only ever grow: no reset pass
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 100.0
        nbytes = side * side * 4
        rows.append({"data_size": nbytes / 2**20, "latency_avg": us, "throughput_avg": nbytes / (us * 1e-6) / 1e9})
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "MB", "latency_unit": "us",
                      "throughput_unit": "GB/s", "metrics": rows}))


if __name__ == "__main__":
    main()
