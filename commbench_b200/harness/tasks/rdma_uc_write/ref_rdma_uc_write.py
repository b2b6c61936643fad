"""Unreliable-connected queue pairs: sends and one-sided writes without acknowledgements.  A send
that finds no posted receive is LOST (the sender still completes), reads and atomics are not
available, writes with an immediate value notify the receiver.  The class below streams a
buffer with plain writes and closes each batch with one write-with-immediate that tells the
receiver how many bytes are valid.  Prints one JSON object.

Reference counterpart: datasets/example007_rdma_send_recv_uc (UC queue pairs, GPU memory as the
buffer on the reference's machine; host memory here), on the package's verbs-style transport.
"""
import json
import time

import numpy as np

from commbench_b200.ops import transport as T

SIZES = [4096, 65536, 1 << 20]
CHUNK = 16384
ROUNDS = 20


class UcStream:
    """Sender and receiver side of a stream over one UC pair (both live in this process)."""

    def __init__(self, ctx: T.Context, nbytes: int):
        self.ctx = ctx
        # --- solution: two UC queue pairs connected to each other (self.tx, self.rx), a source
        #     and a destination buffer of nbytes (uint8) with their memory regions
        self.tx, self.rx = ctx.create_qp(T.UC), ctx.create_qp(T.UC)
        T.connect_pair(self.tx, self.rx)
        self.src = np.zeros(nbytes, dtype=np.uint8)
        self.dst = np.zeros(nbytes, dtype=np.uint8)
        self.m_src, self.m_dst = ctx.reg_mr(self.src), ctx.reg_mr(self.dst)
        # --- end solution

    def push(self, nbytes: int) -> int:
        """Writes src[:nbytes] into dst in CHUNK-sized one-sided writes; the LAST work request is a
        zero-byte write-with-immediate carrying nbytes // CHUNK (the receiver posted one empty
        receive for it).  Returns the immediate value the receiver saw."""
        # --- solution: rx.post_recv(wr, []) first; unsignalled WRITEs for the chunks (flags=0),
        #     then one signalled WRITE_IMM with no data; wait for the sender's completion and the
        #     receiver's RECV_IMM completion
        self.rx.post_recv(1, [])
        off = 0
        while off < nbytes:
            n = min(CHUNK, nbytes - off)
            self.tx.post(T.WRITE, [self.m_src.sge(off, n)], wr_id=2, flags=0,
                         remote_addr=self.m_dst.addr + off, rkey=self.m_dst.rkey)
            off += n
        self.tx.post(T.WRITE_IMM, [], wr_id=3, imm=nbytes // CHUNK, remote_addr=self.m_dst.addr,
                     rkey=self.m_dst.rkey)
        done = self.tx.poll_send(timeout_us=2_000_000)
        got = self.rx.poll_recv(timeout_us=2_000_000)
        if not done or not done[-1].ok or not got or not got[0].ok:
            raise RuntimeError("stream did not complete")
        return got[0].imm
        # --- end solution


def main():
    ok, rows = True, []
    with T.Context(T.LOOPBACK, "lo0") as ctx:
        s = UcStream(ctx, max(SIZES))
        rng = np.random.default_rng(11)
        for n in SIZES:
            s.src[:n] = rng.integers(0, 256, n, dtype=np.uint8)
            s.dst[:] = 0
            ok &= s.push(n) == n // CHUNK and np.array_equal(s.dst[:n], s.src[:n])
            t0 = time.perf_counter()
            for _ in range(ROUNDS):
                s.push(n)
            dt = (time.perf_counter() - t0) / ROUNDS
            rows.append({"data_size": n, "latency_avg": dt * 1e6, "throughput_avg": n / dt / 1e6})
        # what UC does not do
        try:
            s.tx.post(T.READ, [s.m_src.sge(0, 64)], remote_addr=s.m_dst.addr, rkey=s.m_dst.rkey)
            ok = False
        except T.TransportError:
            pass
        s.tx.post(T.SEND, [s.m_src.sge(0, 64)], wr_id=9)          # no receive posted: lost
        ok &= s.tx.poll_send()[0].ok and s.rx.poll_recv(timeout_us=2000) == []
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "B", "latency_unit": "us",
                      "throughput_unit": "MB/s", "metrics": rows}))


if __name__ == "__main__":
    main()
