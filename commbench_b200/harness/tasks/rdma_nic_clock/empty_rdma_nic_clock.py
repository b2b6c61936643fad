"""Read the device's free-running clock and use it to time work requests from the device's
point of view: resolution (smallest non-zero step between back-to-back reads), monotonicity,
agreement with the host's monotonic clock over a known sleep, and the device-clock latency of
a small write.  Prints one JSON object.
"""
import json
import time

import numpy as np

from commbench_b200.ops import transport as T

READS = 2000


class NicClock:
    def __init__(self, ctx: T.Context):
        self.ctx = ctx

    def resolution_ns(self, reads: int) -> tuple[int, bool]:
        """(smallest non-zero difference between consecutive clock reads, monotonic?)."""
        # TODO: ctx.clock_ns() `reads` times; differences must never be negative
        raise NotImplementedError

    def time_write_ns(self, ep: T.Endpoint, mr_src, mr_dst, nbytes: int) -> int:
        """Device-clock nanoseconds from posting one signalled write of nbytes to its completion."""
        # TODO: clock, post WRITE, poll the send completion, clock again
        raise NotImplementedError


def main():
    ok, rows = True, []
    with T.Context(T.LOOPBACK, "lo0") as ctx:
        clk = NicClock(ctx)
        res, mono = clk.resolution_ns(READS)
        ok &= mono and 0 < res < 1_000_000
        h0, d0 = time.monotonic_ns(), ctx.clock_ns()
        time.sleep(0.05)
        h1, d1 = time.monotonic_ns(), ctx.clock_ns()
        ok &= abs((d1 - d0) - (h1 - h0)) < 0.2 * (h1 - h0)          # same rate as the host clock
        a, b = ctx.create_qp(T.RC), ctx.create_qp(T.RC)
        T.connect_pair(a, b)
        src, dst = np.full(65536, 7, dtype=np.uint8), np.zeros(65536, dtype=np.uint8)
        ms, md = ctx.reg_mr(src), ctx.reg_mr(dst)
        for n in (64, 4096, 65536):
            ts = [clk.time_write_ns(a, ms, md, n) for _ in range(200)]
            ok &= all(t > 0 for t in ts) and np.array_equal(dst[:n], src[:n])
            ts.sort()
            rows.append({"data_size": n, "latency_avg": ts[len(ts) // 2] / 1e3,
                         "throughput_avg": n / max(ts[len(ts) // 2], 1) * 1e3, "clock_resolution_ns": res})
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "B", "latency_unit": "us",
                      "throughput_unit": "MB/s", "metrics": rows}))


if __name__ == "__main__":
    main()
