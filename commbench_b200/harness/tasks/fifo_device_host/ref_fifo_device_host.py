"""Queues between the GPU and the CPU, both directions.  Device -> host: many GPU threads push
trigger words into a ring in mapped host memory and a host proxy thread pops them - every id
exactly once.  Host -> device: the CPU pushes task words that a persistent GPU consumer kernel
pops in order.  Every wait is bounded (a full ring nobody drains ends in a status word, not a
hang).  Prints one JSON object.

Reference counterpart: datasets/example003_fifo_device2host (trigger FIFO + proxy thread,
:431-570) and datasets/example005_fifo_host2device (task FIFO + persistent consumer, :364-479).

Run as: python ref_fifo_device_host.py
"""
import json
import time

import torch


class GpuCpuQueues:
    def d2h_round(self, blocks: int, threads: int, per_thread: int, ring: int = 512):
        """Pushes blocks*threads*per_thread ids (1..n) from the GPU through a ring of `ring`
        slots; returns (popped count, checksum of the popped ids, device status word, seconds)."""
        from commbench_b200.ops.util import D2HFifo

        # --- solution: D2HFifo(size=ring); start_proxy(); push_test(..., status=st); synchronize;
        #     wait (bounded, 10 s) until popped() reaches n; stop_proxy() returns
        #     (popped, checksum, span_ns); close()
        f = D2HFifo(size=ring)
        st = torch.zeros(1, dtype=torch.int32, device="cuda")
        f.start_proxy()
        t0 = time.perf_counter()
        f.push_test(blocks, threads, per_thread, status=st)
        torch.cuda.synchronize()
        n = blocks * threads * per_thread
        while f.popped() < n and time.perf_counter() - t0 < 10:
            time.sleep(0.0005)
        dt = time.perf_counter() - t0
        popped, checksum, _ = f.stop_proxy()
        f.close()
        return popped, checksum, int(st.item()), dt
        # --- end solution

    def h2d_round(self, n: int, ring: int = 16):
        """Pushes the words 1000 .. 1000+n-1 from the CPU to a consumer kernel; returns
        (list of words in the order the GPU saw them, device status word, seconds)."""
        from commbench_b200.ops.util import H2DFifo

        # --- solution: H2DFifo(size=ring); launch_consumer(n, timeout_s=5, status=st, stream=s) on
        #     a side stream; push the words; synchronize the stream; column 0 of the result holds
        #     the words
        f = H2DFifo(size=ring)
        st = torch.zeros(1, dtype=torch.int32, device="cuda")
        s = torch.cuda.Stream()
        t0 = time.perf_counter()
        with torch.cuda.stream(s):
            res = f.launch_consumer(n, timeout_s=5.0, status=st, stream=s)
        for i in range(n):
            f.push(1000 + i)
        s.synchronize()
        dt = time.perf_counter() - t0
        words = res[:, 0].tolist()
        f.close()
        return words, int(st.item()), dt
        # --- end solution


def main():
    if not torch.cuda.is_available():
        print(json.dumps({"Correctness": "SKIP", "reason": "no CUDA device", "metrics": []}))
        return
    q = GpuCpuQueues()
    ok, rows = True, []
    for blocks, threads, per in ((1, 32, 4), (4, 256, 16)):
        popped, checksum, status, dt = q.d2h_round(blocks, threads, per)
        n = blocks * threads * per
        ok &= status == 0 and popped == n and checksum == n * (n + 1) // 2
        rows.append({"data_size": n, "latency_avg": dt / n * 1e6, "throughput_avg": n / dt / 1e6})
    words, status, dt = q.h2d_round(200)
    ok &= status == 0 and words == [1000 + i for i in range(200)]
    rows.append({"data_size": 200, "latency_avg": dt / 200 * 1e6, "throughput_avg": 200 / dt / 1e6})
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "items", "latency_unit": "us",
                      "throughput_unit": "Mitems/s", "metrics": rows}))


if __name__ == "__main__":
    main()
