"""Unreliable datagrams: messages of up to one MTU between two UD queue pairs, addressed per
send (address handle + queue key), received behind a 40-byte header.  Prints one JSON object.

Reference counterpart: datasets/example016_rdma_send_recv_ud (UD queue pair, address handle,
qkey, MTU-bounded datagrams :217-237), here on the package's verbs-style transport.
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
        # --- solution: create a UD queue pair (self.qp), make it ready (connect() without a peer),
        #     allocate self.ring (depth * slot bytes, uint8), register it (self.mr) and post one
        #     receive per slot with wr_id = slot index
        self.qp = ctx.create_qp(T.UD)
        self.qp.connect()
        self.ring = np.zeros(depth * slot, dtype=np.uint8)
        self.mr = ctx.reg_mr(self.ring)
        for i in range(depth):
            self.qp.post_recv(i, [self.mr.sge(i * slot, slot)])
        # --- end solution

    def send(self, dest: T.Addr, mr: T.MemoryRegion, nbytes: int):
        # --- solution: post one signalled send of the first nbytes of `mr` to `dest` and wait for
        #     its completion (RuntimeError when it fails or does not arrive within 2 s)
        self.qp.post(T.SEND, [mr.sge(0, nbytes)], wr_id=1, dest=dest)
        got = self.qp.poll_send(timeout_us=2_000_000)
        if not got or not got[0].ok:
            raise RuntimeError("send did not complete")
        # --- end solution

    def receive(self, timeout_us: int = 2_000_000):
        """(payload bytes without the header, sender's queue pair number) of the next datagram,
        or None when nothing arrives in time; the slot is re-posted."""
        # --- solution: poll the receive queue; the payload starts T.UD_HEADER bytes into the slot
        #     named by wr_id and is byte_len - T.UD_HEADER long; copy it out, re-post the slot
        got = self.qp.poll_recv(max_entries=1, timeout_us=timeout_us)
        if not got:
            return None
        c = got[0]
        if not c.ok:
            raise RuntimeError(f"receive failed with status {c.status}")
        base = c.wr_id * self.slot
        data = self.ring[base + T.UD_HEADER:base + c.byte_len].copy()
        self.qp.post_recv(c.wr_id, [self.mr.sge(base, self.slot)])
        return data, c.src_qpn
        # --- end solution


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
