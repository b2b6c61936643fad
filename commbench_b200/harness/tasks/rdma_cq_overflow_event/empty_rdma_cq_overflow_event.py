"""Asynchronous error detection: a completion queue that is too small overflows, the device
raises a CQ error event, and a monitor with a time limit picks it up and acknowledges it.
Reports the detection latency.  Prints one JSON object.

API: ``commbench_b200.ops.transport`` - ``Context.create_cq(depth=)``, ``Context.create_qp(T.RC,
send_cq=, recv_cq=)``, ``Context.get_async_event(timeout_ms=) -> (event, object id) | None``,
``Context.ack_async_event()``, ``Context.clock_ns()``, ``Context.poll_cq(cq, timeout_us=)``,
``T.EVENT_CQ_ERR``.
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
        # TODO: refuse (RuntimeError) while an earlier event is unacknowledged; otherwise wait for
        # an event for at most timeout_ms and remember whether one was taken.
        raise NotImplementedError

    def ack(self):
        # TODO: acknowledge the event taken by wait().
        raise NotImplementedError


def overflow_once(ctx: T.Context, mon: AsyncEventMonitor, src, dst) -> tuple[bool, float]:
    """Creates a tiny completion queue, posts more signalled writes than it holds without polling,
    and returns (detected the right event on the right queue, latency in microseconds)."""
    # TODO:
    #  1. completion queue of CQ_DEPTH entries shared by the send and receive side of queue pair
    #     `a`; a second queue pair `b`; connect them.
    #  2. check that the monitor sees nothing for 5 ms.
    #  3. take ctx.clock_ns(), post CQ_DEPTH + 2 signalled writes src -> dst without polling.
    #  4. wait up to 1 s for the event; latency = clock difference in microseconds.
    #  5. correct iff the event is (T.EVENT_CQ_ERR, that queue), it was acknowledged, and exactly
    #     CQ_DEPTH completions can still be polled.
    #  6. destroy both queue pairs.
    raise NotImplementedError


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
