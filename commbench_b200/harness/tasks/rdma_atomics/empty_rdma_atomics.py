"""Remote atomics from two queue pairs on one 8-byte word: compare-and-swap must have exactly one
winner per round, fetch-and-add must hand out distinct tickets.  Prints one JSON object.

API: ``commbench_b200.ops.transport`` - ``Endpoint.post(T.ATOMIC_CAS, [sge], remote_addr=, rkey=,
compare_add=<expected>, swap=<new>)`` and ``Endpoint.post(T.ATOMIC_FADD, [sge], remote_addr=,
rkey=, compare_add=<addend>)``; the 8-byte local buffer named by the scatter-gather entry
receives the value the word held before the operation.
"""
import json
import time

import numpy as np

from commbench_b200.ops import transport as T

ROUNDS = 200


class AtomicContender:
    """A connected queue pair that fires atomics at a remote word and keeps the value it saw."""

    def __init__(self, ctx: T.Context):
        # TODO: create and connect a pair of RC queue pairs (self.qp is the active side), allocate
        # self.old (one uint64) and register it as self.mr.
        raise NotImplementedError

    def cas(self, target: T.MemoryRegion, expect: int, swap: int):
        # TODO: post a compare-and-swap on the first 8 bytes of `target` (do not wait).
        raise NotImplementedError

    def fetch_add(self, target: T.MemoryRegion, add: int):
        # TODO: post a fetch-and-add on the first 8 bytes of `target` (do not wait).
        raise NotImplementedError

    def result(self) -> int:
        # TODO: wait for the completion (limit 2 s, raise RuntimeError on failure) and return the
        # value the word held before this queue pair's operation.
        raise NotImplementedError


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
