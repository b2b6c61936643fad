"""One-sided write and read plus two-sided send/recv between two reliable-connected queue pairs
of one transport context (loopback device).  Prints one JSON object.

API: ``commbench_b200.ops.transport`` - ``Context.reg_mr(buf)``, ``Context.create_qp(T.RC)``,
``Endpoint.connect(addr)``, ``Endpoint.post(opcode, sges, wr_id=, remote_addr=, rkey=)``,
``Endpoint.post_recv(wr_id, sges)``, ``Endpoint.poll_send / poll_recv(timeout_us=)``,
``MemoryRegion.sge(offset, length)``.
"""
import json
import time

import numpy as np

from commbench_b200.ops import transport as T

SIZES = [64 << 10, 256 << 10, 1 << 20, 4 << 20, 16 << 20]
ITERS = 10


class RdmaEndpoint:
    """A queue pair with its completion queue and one registered buffer."""

    def __init__(self, ctx: T.Context, nbytes: int):
        # TODO: allocate self.buf (uint8, nbytes), register it (self.mr), create an RC queue pair (self.qp).
        raise NotImplementedError

    def connect(self, other: "RdmaEndpoint"):
        # TODO: bring the queue pair to the connected state towards `other`.
        raise NotImplementedError

    def wait(self, recv: bool = False, timeout_us: int = 2_000_000) -> T.Completion:
        # TODO: poll the send (or receive) completion queue; raise TimeoutError when nothing arrives
        # within the limit and RuntimeError on a failed completion; return the completion.
        raise NotImplementedError

    def write(self, peer: "RdmaEndpoint", nbytes: int):
        # TODO: one-sided write of the first nbytes of self.buf into peer.buf; wait for it.
        raise NotImplementedError

    def read(self, peer: "RdmaEndpoint", nbytes: int):
        # TODO: one-sided read of the first nbytes of peer.buf into self.buf; wait for it.
        raise NotImplementedError

    def send(self, nbytes: int):
        # TODO: two-sided send of the first nbytes (do not wait here).
        raise NotImplementedError

    def post_recv(self, nbytes: int):
        # TODO: post a receive for nbytes into self.buf.
        raise NotImplementedError


def main():
    ok, rows = True, []
    with T.Context(T.LOOPBACK, "lo0") as ctx:
        a, b = RdmaEndpoint(ctx, max(SIZES)), RdmaEndpoint(ctx, max(SIZES))
        a.connect(b)
        b.connect(a)
        rng = np.random.default_rng(7)
        for n in SIZES:
            pattern = rng.integers(0, 256, n, dtype=np.uint8)
            a.buf[:n] = pattern
            b.buf[:n] = 0
            ok &= a.write(b, n).byte_len == n and np.array_equal(b.buf[:n], pattern)
            a.buf[:n] = 0
            ok &= a.read(b, n).byte_len == n and np.array_equal(a.buf[:n], pattern)
            b.buf[:n] = 0
            b.post_recv(n)
            a.send(n)
            got = b.wait(recv=True)
            a.wait()
            ok &= got.byte_len == n and got.src_qpn == a.qp.qpn and np.array_equal(b.buf[:n], pattern)
            t0 = time.perf_counter()
            for _ in range(ITERS):
                a.write(b, n)
            dt = (time.perf_counter() - t0) / ITERS
            rows.append({"data_size": n / 2**20, "latency_avg": dt * 1e6, "throughput_avg": n / dt / 1e9})
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "MB", "latency_unit": "us",
                      "throughput_unit": "GB/s", "metrics": rows}))


if __name__ == "__main__":
    main()
