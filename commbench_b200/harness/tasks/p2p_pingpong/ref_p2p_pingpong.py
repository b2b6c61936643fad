"""Round-trip latency of one word between two GPUs through peer memory: one warp per GPU, rank 0
stores a growing counter into rank 1's word with a system-scope release store, rank 1 answers
into rank 0's word, every wait is a bounded acquire poll.  Prints one JSON object.

Reference counterpart: datasets/example073_GPU_p2p_pingpong_latency (``st.release.sys`` /
``ld.acquire.sys`` ping-pong, :30-56).

Launched as: torchrun --nproc-per-node 2 ref_p2p_pingpong.py
"""
from commbench_b200.harness import tasklib

ROUNDS = (200, 2000)


class PingPong:
    def __init__(self, run: tasklib.TaskRun):
        self.ctx = run.ctx

    def round_trip_us(self, rounds: int):
        """Mean round-trip time in microseconds over `rounds` exchanges (None on ranks >= 2)."""
        # --- solution: ops.util.pingpong_latency(ctx, rounds) - collective over the context
        from commbench_b200.ops.util import pingpong_latency

        return pingpong_latency(self.ctx, rounds)
        # --- end solution


def main():
    run = tasklib.start(min_world=2, heap_mb=64)
    pp = PingPong(run)
    ok, rows = True, []
    for n in ROUNDS:
        us = pp.round_trip_us(n)
        again = pp.round_trip_us(n)                  # the words keep growing: a second call must work
        if run.rank < 2:
            ok &= us is not None and again is not None and 0.5 < us < 200.0 and 0.5 < again < 200.0
        rows.append({"data_size": float(n), "latency_avg": float(min(us or 1e9, again or 1e9)),
                     "throughput_avg": 1.0 / max(min(us or 1e9, again or 1e9), 1e-9)})
    run.finish(ok, rows, data_size_unit="rounds", throughput_unit="round trips/us")


if __name__ == "__main__":
    tasklib.guarded(main)
