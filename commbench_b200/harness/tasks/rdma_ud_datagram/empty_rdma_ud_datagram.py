"""Unreliable datagrams: messages of up to one MTU between two UD queue pairs, addressed per
send (address handle + queue key), received behind a 40-byte header.  Prints one JSON object.
"""
import json
import time

import numpy as np

from commbench_b200.ops import transport as T

SIZES = [64, 256, 1024, 4096 - 64]
ROUNDS = 200


class UdEndpoint:
    """A UD queue pair with a receive ring of ``depth`` slots of ``slot`` bytes."""

    def __init__(self, ctx: T.Context, depth: int, slot: int):
        self.ctx, self.depth, self.slot = ctx, depth, slot
        # TODO: create a UD queue pair (self.qp), make it ready (connect() without a peer),
        #       allocate self.ring (depth * slot bytes, uint8), register it (self.mr) and post one
        #       receive per slot with wr_id = slot index
        raise NotImplementedError

    def send(self, dest: T.Addr, mr: T.MemoryRegion, nbytes: int):
        # TODO: post one signalled send of the first nbytes of `mr` to `dest` and wait for
        #       its completion (RuntimeError when it fails or does not arrive within 2 s)
        raise NotImplementedError

    def receive(self, timeout_us: int = 2_000_000):
        """(payload bytes without the header, sender's queue pair number) of the next datagram,
        or None when nothing arrives in time; the slot is re-posted."""
        # TODO: poll the receive queue; the payload starts T.UD_HEADER bytes into the slot
        #       named by wr_id and is byte_len - T.UD_HEADER long; copy it out, re-post the slot
        raise NotImplementedError


def main():
    ok, rows = True, []
    with T.Context(T.LOOPBACK, "lo0") as ctx:
        a = UdEndpoint(ctx, 8, T.UD_HEADER + T.UD_MTU)
        b = UdEndpoint(ctx, 8, T.UD_HEADER + T.UD_MTU)
        out = np.zeros(T.UD_MTU, dtype=np.uint8)
        mo = ctx.reg_mr(out)
        rng = np.random.default_rng(5)
        for n in SIZES:
            t0 = time.perf_counter()
            for _ in range(ROUNDS):
                out[:n] = rng.integers(0, 256, n, dtype=np.uint8)
                a.send(b.qp.addr, mo, n)
                got = b.receive()
                ok &= got is not None and got[1] == a.qp.qpn and np.array_equal(got[0], out[:n])
            dt = (time.perf_counter() - t0) / ROUNDS
            rows.append({"data_size": n, "latency_avg": dt * 1e6, "throughput_avg": n / dt / 1e6})
        # a wrong queue key is dropped without an error on either side
        wrong = T.Addr.unpack(b.qp.addr.pack())
        wrong.qkey ^= 1
        a.send(wrong, mo, 64)
        ok &= b.receive(timeout_us=2000) is None
        # more than one MTU cannot be sent
        big = ctx.reg_mr(np.zeros(T.UD_MTU + 16, dtype=np.uint8))
        try:
            a.send(b.qp.addr, big, T.UD_MTU + 16)
            ok = False
        except T.TransportError:
            pass
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "B", "latency_unit": "us",
                      "throughput_unit": "MB/s", "metrics": rows}))


if __name__ == "__main__":
    main()
