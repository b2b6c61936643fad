"""One-sided writes with an immediate value as the completion notification, received through a
shared receive queue that serves several queue pairs; includes the zero-byte "doorbell" form.
Prints one JSON object.

Reference counterpart: datasets/example008_rdma_write_shared_receive_queue (shared receive queue
+ write / write-with-immediate :202-292), datasets/example011_rdma_write_rc_with_imm (notification
latency :153-183) and datasets/example013_rdma_write_zero_message (zero-byte form :149-198), here on
the package's verbs-style transport.
"""
import json
import time

import numpy as np

from commbench_b200.ops import transport as T

N_SENDERS = 3
SIZES = [0, 4096, 1 << 20, 16 << 20]
ROUNDS = 50


class Receiver:
    """``n`` queue pairs that share one receive queue and one completion queue, and one buffer
    that the senders write into (sender i owns the i-th slice)."""

    def __init__(self, ctx: T.Context, n: int, slice_bytes: int):
        self.ctx, self.n, self.slice_bytes = ctx, n, slice_bytes
        self.buf = np.zeros(n * slice_bytes, dtype=np.uint8)
        self.mr = ctx.reg_mr(self.buf)
        # --- solution: create self.srq and self.cq, then n RC queue pairs (self.qps) that use both;
        #     keep self.posted = 0 (receives posted so far)
        self.srq = ctx.create_srq(64)
        self.cq = ctx.create_cq(256)
        self.qps = [ctx.create_qp(T.RC, send_cq=self.cq, recv_cq=self.cq, srq=self.srq) for _ in range(n)]
        self.posted = 0
        # --- end solution

    def post_receives(self, count: int):
        # --- solution: post `count` empty receives (no buffer: the data lands through the write)
        #     to the shared queue, with increasing wr_id
        for _ in range(count):
            self.ctx.post_srq_recv(self.srq, self.posted, [])
            self.posted += 1
        # --- end solution

    def wait_notifications(self, count: int, timeout_s: float = 5.0) -> list[tuple[int, int, int]]:
        """[(queue pair number it arrived on, immediate value, bytes written)] for `count`
        notifications; RuntimeError when they do not all arrive in time."""
        # --- solution: poll self.cq until `count` completions with opcode T.RECV_IMM are in
        out, deadline = [], time.monotonic() + timeout_s
        while len(out) < count:
            for c in self.ctx.poll_cq(self.cq, timeout_us=100_000):
                if not c.ok:
                    raise RuntimeError(f"completion failed with status {c.status}")
                if c.opcode == T.RECV_IMM:
                    out.append((c.qpn, c.imm, c.byte_len))
            if time.monotonic() > deadline:
                raise RuntimeError("notifications did not arrive")
        return out
        # --- end solution


class Sender:
    def __init__(self, ctx: T.Context, index: int, nbytes: int):
        self.index = index
        self.buf = np.full(nbytes, index + 1, dtype=np.uint8)
        self.mr = ctx.reg_mr(self.buf)
        self.qp = ctx.create_qp(T.RC)

    def notify(self, rx: Receiver, nbytes: int, imm: int):
        # --- solution: one signalled write-with-immediate of the first nbytes of self.buf into
        #     this sender's slice of rx.buf (nbytes may be 0: then no scatter-gather entry at all);
        #     wait for the send completion (RuntimeError on failure)
        sges = [self.mr.sge(0, nbytes)] if nbytes else []
        self.qp.post(T.WRITE_IMM, sges, wr_id=7, imm=imm,
                     remote_addr=rx.mr.addr + self.index * rx.slice_bytes, rkey=rx.mr.rkey)
        got = self.qp.poll_send(timeout_us=5_000_000)
        if not got or not got[0].ok:
            raise RuntimeError("write did not complete")
        # --- end solution


def main():
    ok, rows = True, []
    with T.Context(T.LOOPBACK, "lo0") as ctx:
        rx = Receiver(ctx, N_SENDERS, max(SIZES))
        senders = [Sender(ctx, i, max(SIZES)) for i in range(N_SENDERS)]
        for s, q in zip(senders, rx.qps):
            T.connect_pair(s.qp, q)
        for n in SIZES:
            rx.buf[:] = 0
            rx.post_receives(N_SENDERS)
            for s in senders:
                s.notify(rx, n, imm=1000 * s.index + 5)
            got = sorted(rx.wait_notifications(N_SENDERS))
            want = sorted((q.qpn, 1000 * s.index + 5, n) for s, q in zip(senders, rx.qps))
            ok &= got == want
            for s in senders:
                sl = rx.buf[s.index * rx.slice_bytes:s.index * rx.slice_bytes + max(n, 1)]
                ok &= bool((sl[:n] == s.index + 1).all()) and (n > 0 or sl[0] == 0)
            t0 = time.perf_counter()
            for r in range(ROUNDS):
                rx.post_receives(1)
                senders[0].notify(rx, n, imm=r)
                ok &= rx.wait_notifications(1)[0][1] == r
            dt = (time.perf_counter() - t0) / ROUNDS
            rows.append({"data_size": n / 2**20, "latency_avg": dt * 1e6,
                         "throughput_avg": n / dt / 1e9 if n else 0.0})
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "MB", "latency_unit": "us",
                      "throughput_unit": "GB/s", "metrics": rows}))


if __name__ == "__main__":
    main()
