"""Two ways of shaping one write request: inline payloads (copied into the work request, no local
key, up to the queue pair's inline limit) and a scatter-gather list that gathers several
non-contiguous registered pieces into one contiguous remote range.  Prints one JSON object.

Reference counterpart: datasets/example014_rdma_write_inline (inline flag, query of the limit
:205-272) and datasets/example019_rdma_write_scatter_gather_lists (one write gathering kNumSge
regions :227-256), here on the package's verbs-style transport.
"""
import json
import time

import numpy as np

from commbench_b200.ops import transport as T

INLINE_LIMIT = 256
NUM_SGE = 8
PIECE_SIZES = [4 << 10, 64 << 10, 1 << 20]
ROUNDS = 20


class Writer:
    def __init__(self, ctx: T.Context):
        self.ctx = ctx
        # --- solution: a connected pair of RC queue pairs (self.qp active, self.far passive) whose
        #     inline limit is INLINE_LIMIT bytes
        self.qp = ctx.create_qp(T.RC, max_inline=INLINE_LIMIT)
        self.far = ctx.create_qp(T.RC, max_inline=INLINE_LIMIT)
        T.connect_pair(self.qp, self.far)
        # --- end solution

    def _done(self):
        got = self.qp.poll_send(timeout_us=5_000_000)
        if not got or not got[0].ok:
            raise RuntimeError("write did not complete")
        return got[0]

    def inline_limit(self) -> int:
        # --- solution: the queue pair's inline limit as the transport reports it
        return self.qp.max_inline
        # --- end solution

    def write_inline(self, payload: np.ndarray, dst: T.MemoryRegion):
        """Writes an UNREGISTERED host array into dst; the transport refuses (TransportError)
        payloads above the limit."""
        # --- solution: scatter-gather entry (address, length, 0) taken with T.buffer_address,
        #     flags SIGNALED | INLINE; wait for the completion
        addr, n = T.buffer_address(payload)
        self.qp.post(T.WRITE, [(addr, n, 0)], flags=T.SIGNALED | T.INLINE, remote_addr=dst.addr, rkey=dst.rkey)
        return self._done()
        # --- end solution

    def write_gather(self, pieces: list[T.MemoryRegion], dst: T.MemoryRegion):
        # --- solution: ONE write whose scatter-gather list names every piece in order; returns
        #     the completion (its byte_len is the total)
        self.qp.post(T.WRITE, [p.sge() for p in pieces], remote_addr=dst.addr, rkey=dst.rkey)
        return self._done()
        # --- end solution


def main():
    ok, rows = True, []
    with T.Context(T.LOOPBACK, "lo0") as ctx:
        w = Writer(ctx)
        ok &= w.inline_limit() == INLINE_LIMIT
        small_dst = np.zeros(INLINE_LIMIT, dtype=np.uint8)
        md = ctx.reg_mr(small_dst)
        for n in (1, 64, INLINE_LIMIT):
            payload = np.arange(n, dtype=np.uint8) + 3
            small_dst[:] = 0
            ok &= w.write_inline(payload, md).byte_len == n and np.array_equal(small_dst[:n], payload)
        try:
            w.write_inline(np.zeros(INLINE_LIMIT + 1, dtype=np.uint8), md)
            ok = False
        except T.TransportError:
            pass
        t0 = time.perf_counter()
        for _ in range(200):
            w.write_inline(np.zeros(64, dtype=np.uint8), md)
        inline_us = (time.perf_counter() - t0) / 200 * 1e6
        rows.append({"data_size": 64 / 2**20, "latency_avg": inline_us, "throughput_avg": 64 / inline_us / 1e3})
        for size in PIECE_SIZES:
            parts = [np.full(size + 16 * i, i + 1, dtype=np.uint8) for i in range(NUM_SGE)]
            mrs = [ctx.reg_mr(p) for p in parts]
            total = sum(p.size for p in parts)
            dst = np.zeros(total, dtype=np.uint8)
            mdst = ctx.reg_mr(dst)
            ok &= w.write_gather(mrs, mdst).byte_len == total and np.array_equal(dst, np.concatenate(parts))
            t0 = time.perf_counter()
            for _ in range(ROUNDS):
                w.write_gather(mrs, mdst)
            dt = (time.perf_counter() - t0) / ROUNDS
            rows.append({"data_size": total / 2**20, "latency_avg": dt * 1e6, "throughput_avg": total / dt / 1e9})
            for m in mrs + [mdst]:
                ctx.dereg_mr(m)
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "MB", "latency_unit": "us",
                      "throughput_unit": "GB/s", "metrics": rows}))


if __name__ == "__main__":
    main()
