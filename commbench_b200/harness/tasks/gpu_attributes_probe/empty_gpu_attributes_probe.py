"""List what the GPU is: name, compute capability, SM count, memory, L2, shared memory per block
and per SM, registers, clocks, bus width, cooperative launch, unified addressing - one JSON
object a scheduler or an autotuner can read - and derive two numbers from it the way the
rest of the package does: resident 512-thread CTAs per SM by registers at 64 registers per
thread, and the nominal HBM bandwidth from the memory clock and the bus width.
Prints one JSON object.

Run as: python ref_gpu_attributes_probe.py
"""
import json
import time

import torch


class GpuAttributes:
    def query(self, device: int = 0) -> dict:
        """The attribute dictionary of the package's probe (``ops.util.device_attributes``)."""
        # TODO: one call
        raise NotImplementedError

    def derived(self, a: dict) -> dict:
        """{"ctas_per_sm_by_regs": regs_per_sm // (512 * 64),
            "nominal_hbm_gbs": 2 (DDR) * mem_clock_khz * 1e3 * mem_bus_bits / 8 / 1e9}"""
        # TODO: plain arithmetic on the attributes
        raise NotImplementedError


def main():
    if not torch.cuda.is_available():
        print(json.dumps({"Correctness": "SKIP", "reason": "no CUDA device", "metrics": []}))
        return
    g = GpuAttributes()
    a = g.query(0)
    p = torch.cuda.get_device_properties(0)
    ok = a is not None and a["sm_count"] == p.multi_processor_count and a["warp_size"] == 32
    ok = ok and a["global_mem_bytes"] == p.total_memory
    ok = ok and a["compute_capability"] == f"{p.major}.{p.minor}" and a["name"] == p.name
    d = g.derived(a) if ok else {}
    ok = ok and d.get("ctas_per_sm_by_regs") == a["regs_per_sm"] // 32768
    ok = ok and abs(d.get("nominal_hbm_gbs", 0) - 2e3 * a["mem_clock_khz"] * a["mem_bus_bits"] / 8e9) < 1e-6
    t0 = time.perf_counter()
    for _ in range(50):
        g.query(0)
    dt = (time.perf_counter() - t0) / 50
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "query", "latency_unit": "us",
                      "throughput_unit": "kquery/s", "attributes": a if ok else None,
                      "metrics": [{"data_size": 1, "latency_avg": dt * 1e6, "throughput_avg": 1e-3 / dt}]}))


if __name__ == "__main__":
    main()
