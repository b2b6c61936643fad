"""Asynchronous error detection: a completion queue that is too small overflows, the device
raises a CQ error event, and a monitor with a time limit picks it up and acknowledges it.
Reports the detection latency.  Prints one JSON object.

Same exercise as the reference's datasets/example026_rdma_ibv_get_async_event
(monitor with non-blocking wait + mandatory ack :75-125, detection-latency trials :537-575), on
the package's verbs-style transport.
"""
import json

import numpy as np

from commbench_b200.ops import transport as T

TRIALS = 20
CQ_DEPTH = 2


class AsyncEventMonitor:
    """Waits for device events with a time limit; every event taken must be acknowledged."""

    def __init__(self, ctx: T.Context):
        self.ctx = ctx
        self.pending_ack = False

    def wait(self, timeout_ms: int):
        """(event, object id) or None when the limit passes."""
        if self.pending_ack:
            raise RuntimeError("previous event was not acknowledged")
        ev = self.ctx.get_async_event(timeout_ms=timeout_ms)
        self.pending_ack = ev is not None
        return ev

    def ack(self):
        self.ctx.ack_async_event()
        self.pending_ack = False


def overflow_once(ctx: T.Context, mon: AsyncEventMonitor, src, dst) -> tuple[bool, float]:
    """Creates a tiny completion queue, posts more signalled writes than it holds without polling,
    and returns (detected the right event on the right queue, latency in microseconds)."""
    cq = ctx.create_cq(depth=CQ_DEPTH)
    a = ctx.create_qp(T.RC, send_cq=cq, recv_cq=cq)
    b = ctx.create_qp(T.RC)
    T.connect_pair(a, b)
    quiet = mon.wait(5) is None                      # nothing pending before the overflow
    t0 = ctx.clock_ns()
    for i in range(CQ_DEPTH + 2):
        a.post(T.WRITE, [src.sge()], wr_id=i, remote_addr=dst.addr, rkey=dst.rkey)
    ev = mon.wait(1000)
    latency_us = (ctx.clock_ns() - t0) / 1e3
    good = quiet and ev == (T.EVENT_CQ_ERR, cq)
    if ev is not None:
        mon.ack()
    good &= len(ctx.poll_cq(cq, timeout_us=1000)) == CQ_DEPTH   # what fitted is still readable
    a.destroy()
    b.destroy()
    return good, latency_us


def main():
    ok, lat = True, []
    with T.Context(T.LOOPBACK, "lo0") as ctx:
        s, d = np.ones(8, dtype=np.uint8), np.zeros(8, dtype=np.uint8)
        src, dst = ctx.reg_mr(s), ctx.reg_mr(d)
        mon = AsyncEventMonitor(ctx)
        for _ in range(TRIALS):
            good, us = overflow_once(ctx, mon, src, dst)
            ok &= good
            lat.append(us)
        ok &= mon.wait(5) is None                    # acknowledged events do not come back
    avg = sum(lat) / len(lat)
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "events", "latency_unit": "us",
                      "throughput_unit": "events/s",
                      "metrics": [{"data_size": TRIALS, "latency_avg": avg, "latency_max": max(lat),
                                   "throughput_avg": 1e6 / avg}]}))


if __name__ == "__main__":
    main()
