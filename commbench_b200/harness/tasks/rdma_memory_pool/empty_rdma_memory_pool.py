"""A pool over ONE registered region: registering memory is expensive, so a communication layer
registers one large buffer once and hands out aligned slices from a stack allocator; every slice
shares the region's keys.  Correctness plus the cost of a slice against a fresh registration.
Prints one JSON object.
"""
import json
import time

import numpy as np

from commbench_b200.ops import transport as T

POOL_BYTES = 8 << 20
ALIGN = 256


class MemoryPool:
    """``alloc`` returns (address, length, local key) of the next aligned slice; ``release``
    gives back the most recent ``count`` slices (a stack)."""

    def __init__(self, ctx: T.Context, nbytes: int, align: int = ALIGN):
        self.ctx, self.align = ctx, align
        # TODO: allocate self.buf (uint8, nbytes), register it ONCE (self.mr), start with an
        #       empty stack of slice starts (self.marks) and self.top = first aligned ADDRESS offset
        raise NotImplementedError

    @property
    def used(self) -> int:
        """Bytes between the first slice and the top of the stack (0 when empty)."""
        # TODO: implement
        raise NotImplementedError

    def alloc(self, nbytes: int) -> tuple[int, int, int]:
        # TODO: the slice starts at the current top (an aligned absolute address), the
        #       top moves up by nbytes rounded up to the alignment; T.TransportError when the
        #       region is exhausted or nbytes <= 0
        raise NotImplementedError

    def release(self, count: int = 1):
        # TODO: pop `count` slices; T.TransportError when fewer are outstanding
        raise NotImplementedError

    def view(self, sge: tuple[int, int, int]) -> np.ndarray:
        """The numpy view of a slice (for filling and checking)."""
        off = sge[0] - self.mr.addr
        return self.buf[off:off + sge[1]]


def main():
    ok = True
    with T.Context(T.LOOPBACK, "lo0") as ctx:
        pool = MemoryPool(ctx, POOL_BYTES)
        a, b = ctx.create_qp(T.RC), ctx.create_qp(T.RC)
        T.connect_pair(a, b)
        s1, s2, s3 = pool.alloc(1000), pool.alloc(1), pool.alloc(4096)
        ok &= all(s[0] % ALIGN == 0 and s[2] == pool.mr.lkey for s in (s1, s2, s3))
        ok &= s2[0] == s1[0] + 1024 and s3[0] == s2[0] + ALIGN and pool.used == 1024 + ALIGN + 4096
        # slices are usable as sources and (through the region's remote key) as targets
        pool.view(s1)[:] = 7
        a.post(T.WRITE, [s1], remote_addr=s3[0], rkey=pool.mr.rkey)
        got = a.poll_send(timeout_us=2_000_000)
        ok &= bool(got) and got[0].ok and bool((pool.view(s3)[:1000] == 7).all()) and pool.view(s3)[1000] == 0
        pool.release()
        ok &= pool.alloc(50)[0] == s3[0]                     # the stack re-uses the released slice
        pool.release(3)
        ok &= pool.used == 0
        for bad in (lambda: pool.release(), lambda: pool.alloc(POOL_BYTES + 1), lambda: pool.alloc(0)):
            try:
                bad()
                ok = False
            except T.TransportError:
                pass
        n = 2000
        t0 = time.perf_counter()
        for _ in range(n):
            pool.alloc(4096)
        pool.release(n)
        slice_us = (time.perf_counter() - t0) / n * 1e6
        scratch = np.zeros(4096, dtype=np.uint8)
        t0 = time.perf_counter()
        for _ in range(200):
            ctx.dereg_mr(ctx.reg_mr(scratch))
        reg_us = (time.perf_counter() - t0) / 200 * 1e6
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "B", "latency_unit": "us",
                      "throughput_unit": "Mops/s", "register_latency_us": reg_us,
                      "metrics": [{"data_size": 4096, "latency_avg": slice_us, "throughput_avg": 1.0 / slice_us}]}))


if __name__ == "__main__":
    main()
