"""Remote atomics from two queue pairs on one 8-byte word: compare-and-swap must have exactly one
winner per round, fetch-and-add must hand out distinct tickets.  Prints one JSON object.

Same exercise as the reference's datasets/example024_rdma_atomic_cmp_swp (exactly-one-winner check,
:1-16) and datasets/example025_rdma_atomic_fetch_add ({0,1} check, :1-16), on the package's
verbs-style transport.
"""
import json
import time

import numpy as np

from commbench_b200.ops import transport as T

ROUNDS = 200


class AtomicContender:
    """A connected queue pair that fires atomics at a remote word and keeps the value it saw."""

    def __init__(self, ctx: T.Context):
        self.qp, self.far = ctx.create_qp(T.RC), ctx.create_qp(T.RC)
        T.connect_pair(self.qp, self.far)
        self.old = np.zeros(1, dtype=np.uint64)
        self.mr = ctx.reg_mr(self.old)

    def cas(self, target: T.MemoryRegion, expect: int, swap: int):
        self.qp.post(T.ATOMIC_CAS, [self.mr.sge()], remote_addr=target.addr, rkey=target.rkey,
                     compare_add=expect, swap=swap)

    def fetch_add(self, target: T.MemoryRegion, add: int):
        self.qp.post(T.ATOMIC_FADD, [self.mr.sge()], remote_addr=target.addr, rkey=target.rkey,
                     compare_add=add)

    def result(self) -> int:
        got = self.qp.poll_send(timeout_us=2_000_000)
        if not got or not got[0].ok:
            raise RuntimeError("atomic did not complete")
        return int(self.old[0])


def main():
    ok = True
    with T.Context(T.LOOPBACK, "lo0") as ctx:
        word = np.zeros(1, dtype=np.uint64)
        target = ctx.reg_mr(word)
        p, q = AtomicContender(ctx), AtomicContender(ctx)
        t0 = time.perf_counter()
        for r in range(ROUNDS):
            word[0] = 0
            p.cas(target, 0, 1000 + r)
            q.cas(target, 0, 2000 + r)
            seen = sorted((p.result(), q.result()))
            winner = int(word[0])
            ok &= winner in (1000 + r, 2000 + r) and seen == [0, winner]
        cas_us = (time.perf_counter() - t0) / (2 * ROUNDS) * 1e6
        word[0] = 0
        tickets = []
        t0 = time.perf_counter()
        for r in range(ROUNDS):
            p.fetch_add(target, 1)
            q.fetch_add(target, 1)
            tickets += [p.result(), q.result()]
        fadd_us = (time.perf_counter() - t0) / (2 * ROUNDS) * 1e6
        ok &= sorted(tickets) == list(range(2 * ROUNDS)) and int(word[0]) == 2 * ROUNDS
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "B", "latency_unit": "us",
                      "throughput_unit": "Mops/s",
                      "metrics": [{"data_size": 8, "latency_avg": cas_us, "throughput_avg": 1.0 / cas_us},
                                  {"data_size": 8, "latency_avg": fadd_us, "throughput_avg": 1.0 / fadd_us}]}))


if __name__ == "__main__":
    main()
