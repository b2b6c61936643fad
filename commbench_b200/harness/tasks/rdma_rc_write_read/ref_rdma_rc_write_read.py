"""One-sided write and read plus two-sided send/recv between two reliable-connected queue pairs
of one transport context (loopback device).  Prints one JSON object.

Same exercise as the reference's datasets/example002_rdma_loopback/ib/empty_rdma_loopback.cpp:142-390
(endpoint set-up, write / read / send / recv, completion polling with a time limit), on the
package's verbs-style transport instead of raw libibverbs.
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
        self.ctx = ctx
        self.buf = np.zeros(nbytes, dtype=np.uint8)
        self.mr = ctx.reg_mr(self.buf)
        self.qp = ctx.create_qp(T.RC)

    def connect(self, other: "RdmaEndpoint"):
        self.qp.connect(other.qp.addr)

    def wait(self, recv: bool = False, timeout_us: int = 2_000_000) -> T.Completion:
        got = self.qp.poll_recv(timeout_us=timeout_us) if recv else self.qp.poll_send(timeout_us=timeout_us)
        if not got:
            raise TimeoutError("no completion within the time limit")
        if not got[0].ok:
            raise RuntimeError(f"work request {got[0].wr_id} failed with status {got[0].status}")
        return got[0]

    def write(self, peer: "RdmaEndpoint", nbytes: int):
        self.qp.post(T.WRITE, [self.mr.sge(0, nbytes)], wr_id=1, remote_addr=peer.mr.addr, rkey=peer.mr.rkey)
        return self.wait()

    def read(self, peer: "RdmaEndpoint", nbytes: int):
        self.qp.post(T.READ, [self.mr.sge(0, nbytes)], wr_id=2, remote_addr=peer.mr.addr, rkey=peer.mr.rkey)
        return self.wait()

    def send(self, nbytes: int):
        self.qp.post(T.SEND, [self.mr.sge(0, nbytes)], wr_id=3)

    def post_recv(self, nbytes: int):
        self.qp.post_recv(4, [self.mr.sge(0, nbytes)])


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
