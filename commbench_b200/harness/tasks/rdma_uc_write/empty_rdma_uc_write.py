"""Unreliable-connected queue pairs: sends and one-sided writes without acknowledgements.  A send
that finds no posted receive is LOST (the sender still completes), reads and atomics are not
available, writes with an immediate value notify the receiver.  The class below streams a
buffer with plain writes and closes each batch with one write-with-immediate that tells the
receiver how many bytes are valid.  Prints one JSON object.
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
        # TODO: two UC queue pairs connected to each other (self.tx, self.rx), a source
        #       and a destination buffer of nbytes (uint8) with their memory regions
        raise NotImplementedError

    def push(self, nbytes: int) -> int:
        """Writes src[:nbytes] into dst in CHUNK-sized one-sided writes; the LAST work request is a
        zero-byte write-with-immediate carrying nbytes // CHUNK (the receiver posted one empty
        receive for it).  Returns the immediate value the receiver saw."""
        # TODO: rx.post_recv(wr, []) first; unsignalled WRITEs for the chunks (flags=0),
        #       then one signalled WRITE_IMM with no data; wait for the sender's completion and the
        #       receiver's RECV_IMM completion
        raise NotImplementedError


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
