"""All-reduce between two ranks that are connected only by a transport (another node): every
rank PUTs its vector into the peer's receive window, bumps the peer's signal counter with a
remote fetch-and-add, flushes (both work requests completed), waits until its own counter says
the peer's vector has landed, and adds.  Repeated calls reuse the windows: the counter counts
rounds.  Prints one JSON object.

Reference counterpart: datasets/example092_nccl_device_api_internode_allreduce (put with a
signal increment, wait on the signal, flush, local add, :47-87), expressed on work requests of
the package's verbs-style transport instead of a vendor's device API.
"""
import json
import time

import numpy as np

from commbench_b200.ops import transport as T

SIZES = [1024, 65536, 1 << 20]          # float32 elements
ROUNDS = 10


class PutSignalAllReduce:
    def __init__(self, ctx: T.Context, ep: T.Endpoint, numel: int):
        self.ctx, self.ep, self.numel = ctx, ep, numel
        # --- solution: send and receive vectors (float32), a signal counter and a scratch word
        #     (uint64, the fetch-and-add returns the old value there), all registered; round = 0
        self.send = np.zeros(numel, dtype=np.float32)
        self.recv = np.zeros(numel, dtype=np.float32)
        self.signal = np.zeros(1, dtype=np.uint64)
        self.scratch = np.zeros(1, dtype=np.uint64)
        self.m_send, self.m_recv = ctx.reg_mr(self.send), ctx.reg_mr(self.recv)
        self.m_sig, self.m_scr = ctx.reg_mr(self.signal), ctx.reg_mr(self.scratch)
        self.round = 0
        # --- end solution
        self.peer = None

    def window(self):
        """(receive-window address, its key, signal-counter address, its key) for the peer."""
        # --- solution: addresses and remote keys of self.recv and self.signal
        return (self.m_recv.addr, self.m_recv.rkey, self.m_sig.addr, self.m_sig.rkey)
        # --- end solution

    def connect_window(self, peer_window):
        self.peer = tuple(peer_window)

    def start(self, x, n: int):
        """Posts the put of x[:n] and the signal increment (does not wait)."""
        # --- solution: copy x into self.send, round += 1, one WRITE of n floats into the peer's
        #     window, one ATOMIC_FADD of 1 on the peer's counter (8-byte scratch as the local buffer)
        self.send[:n] = x[:n]
        raddr, rkey, saddr, skey = self.peer
        self.round += 1
        self.ep.post(T.WRITE, [self.m_send.sge(0, 4 * n)], wr_id=2 * self.round, remote_addr=raddr,
                     rkey=rkey)
        self.ep.post(T.ATOMIC_FADD, [self.m_scr.sge()], wr_id=2 * self.round + 1, remote_addr=saddr,
                     rkey=skey, compare_add=1)
        # --- end solution

    def finish(self, n: int, timeout_s: float = 5.0):
        """Flush, wait for the peer's signal (bounded), return send[:n] + recv[:n]."""
        # --- solution: poll both send completions (fail on a bad status), then spin - with a
        #     deadline - until self.signal[0] >= self.round; raise T.TransportError on a time-out
        deadline = time.monotonic() + timeout_s
        done = 0
        while done < 2:
            for c in self.ep.poll_send(timeout_us=100_000):
                if not c.ok:
                    raise T.TransportError(f"put failed with status {c.status}")
                done += 1
            if time.monotonic() > deadline:
                raise T.TransportError("flush timed out")
        while int(self.signal[0]) < self.round:
            if time.monotonic() > deadline:
                raise T.TransportError("the peer's signal never arrived")
            time.sleep(0)
        return self.send[:n] + self.recv[:n]
        # --- end solution


def main():
    ok, rows = True, []
    with T.Context(T.LOOPBACK, "lo0") as ctx:
        a, b = ctx.create_qp(T.RC), ctx.create_qp(T.RC)
        T.connect_pair(a, b)
        ra, rb = PutSignalAllReduce(ctx, a, max(SIZES)), PutSignalAllReduce(ctx, b, max(SIZES))
        ra.connect_window(rb.window())
        rb.connect_window(ra.window())
        rng = np.random.default_rng(2)
        for n in SIZES:
            xa, xb = rng.random(n, dtype=np.float32), rng.random(n, dtype=np.float32)
            t0 = time.perf_counter()
            for _ in range(ROUNDS):
                ra.start(xa, n)
                rb.start(xb, n)
                ya, yb = ra.finish(n), rb.finish(n)
            dt = (time.perf_counter() - t0) / ROUNDS
            ok &= np.array_equal(ya, yb) and np.allclose(ya, xa + xb)
            rows.append({"data_size": 4 * n, "latency_avg": dt * 1e6, "throughput_avg": 4 * n / dt / 1e6})
        lonely = PutSignalAllReduce(ctx, a, 8)             # a peer that never answers: bounded wait
        lonely.connect_window(rb.window())
        lonely.start(np.ones(8, dtype=np.float32), 8)
        try:
            lonely.finish(8, timeout_s=0.3)
            ok = False
        except T.TransportError:
            pass
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "B", "latency_unit": "us",
                      "throughput_unit": "MB/s", "metrics": rows}))


if __name__ == "__main__":
    main()
