#!/usr/bin/env python
"""Headline benchmark: one tensor-parallel MLP step built from the fused kernels.

    x_local [T/N, H] --(all-gather -> GEMM, one kernel)--> h [T, I/N]
                     --(GEMM -> reduce-scatter, one kernel)--> y_local [T/N, H]

with T=8192 tokens, H=8192, I=28672 (the tensor-parallel shapes of the fused-GEMM
configuration: AG->GEMM M=8192,K=8192,N=28672/N and GEMM->RS M=8192,K=28672/N,N=8192),
bf16, random-init weights N(0, 0.02), synthetic activations N(0, 1).  Total work is fixed
as N grows (strong scaling).  `value` is the whole-job TFLOP/s of the fused step; the same
line also carries the speed-up over the unfused NCCL + cuBLAS composition measured in the
same process, the fraction of the roofline, and the all-reduce bus bandwidth.

Launch: ``python bench.py`` (1 GPU) or
``python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1
--master-port P bench.py --gpus N --steps K --warmup W``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def reference_arm() -> int:
    # The reference is a benchmark suite without a package definition (no setup.py /
    # pyproject.toml) and its solution sources (ref_*) are not part of the checkout: the
    # example files are templates whose kernels are TODO bodies.
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference is not installable (pip: neither setup.py nor pyproject.toml) "
                       "and ships only empty_* templates with TODO kernel bodies, no ref_* solutions",
    }))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons of the local GPU with NVML (read-only)."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thr is not None:
            self._thr.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def load_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p["bf16_tflops_sustained"],
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    except Exception:
        return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0,
                "source": "fallback"}


NVLINK_GBS = 770.0        # measured peer copy, per direction per GPU ("of measured")
NVLINK_LINK_GBS = 900.0   # NVLink 5 link rate, per direction per GPU ("of link")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--intermediate", type=int, default=28672)
    ap.add_argument("--skip-extras", action="store_true",
                    help="only the headline numbers (no all-reduce bandwidth line)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and rank == 0:
        print(f"[bench] note: --gpus {args.gpus} but WORLD_SIZE={world}; using {world}",
              file=sys.stderr)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from commbench_b200 import _native
    from commbench_b200.models.tp_mlp import TPMLP
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import CommContext

    if not _native.available():
        from commbench_b200 import _build

        if rank == 0:
            _build.build()
        if world > 1:
            dist.barrier()
    T, H, I = args.tokens, args.hidden, args.intermediate
    ctx = CommContext(heap_bytes=3 << 30)
    mlp = TPMLP(ctx, H, I, T, seed=0)
    Tl = T // world
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    x_local = torch.randn(Tl, H, device=dev, generator=g).bfloat16()
    x_host = torch.empty(Tl, H, dtype=torch.bfloat16).pin_memory()
    x_host.copy_(x_local)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        """K steps between two events, bracketed by barrier+synchronize; max over ranks (ms)."""
        for _ in range(warmup):
            fn()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # correctness of the fused step against the unfused composition, once, before timing
    y_f = mlp.forward(x_local).float().clone()
    ctx.check_status()
    y_u = mlp.forward_unfused(x_local).float()
    rel = ((y_f - y_u).abs().max() / (y_u.abs().max() + 1e-9)).item()

    sampler = ClockSampler(local_rank)
    sampler.start()
    total_ms = timed(lambda: mlp.forward(x_local), args.steps, args.warmup)
    clocks = sampler.stop()
    ctx.check_status()
    ms_step = total_ms / args.steps
    flops = mlp.flops(T)
    value = flops / (ms_step * 1e-3) / 1e12

    base_ms = timed(lambda: mlp.forward_unfused(x_local), args.steps, args.warmup) / args.steps
    e2e_ms = timed(lambda: mlp.forward_host(x_host), args.steps, args.warmup) / args.steps
    e2e_base_ms = timed(lambda: mlp.forward_host(x_host, fused=False), args.steps,
                        args.warmup) / args.steps
    ctx.check_status()

    peaks = load_peaks()
    per_rank_flops_half = flops / world / 2.0
    ag_bytes = (world - 1) / world * T * H * 2.0
    rs_bytes = (world - 1) / world * T * H * 2.0

    def roof(peak_tflops, link_gbs=NVLINK_GBS):
        t1 = max(per_rank_flops_half / (peak_tflops * 1e12), ag_bytes / (link_gbs * 1e9))
        t2 = max(per_rank_flops_half / (peak_tflops * 1e12), rs_bytes / (link_gbs * 1e9))
        return (t1 + t2) * 1e3

    extras = {}
    if not args.skip_extras:
        # All-reduce bus bandwidth, bf16, in place on symmetric tensors, through the library's
        # own selector and default grids (`algo="auto"`).  With one rank there is nothing to
        # reduce over a link: the entries are null.
        for mb in (64, 256):
            n = mb * (1 << 20) // 2
            nbytes = n * 2
            if world == 1:
                extras[f"allreduce_{mb}MB"] = {"algo": None, "ms": None, "busbw_gbs": None,
                                               "nccl_ms": None, "nccl_busbw_gbs": None}
                continue
            t, _ = ctx.empty((n,), torch.bfloat16)
            t.fill_(0.001)
            sync_all()
            algo = coll.plan_all_reduce(ctx, nbytes, True)["algo"]
            ms = timed(lambda: coll.all_reduce(ctx, t), 10, 3) / 10
            u = torch.full((n,), 0.001, dtype=torch.bfloat16, device=dev)
            nccl_ms = timed(lambda: dist.all_reduce(u), 10, 3) / 10
            factor = 2.0 * (world - 1) / world
            bus = factor * nbytes / (ms * 1e-3) / 1e9
            extras[f"allreduce_{mb}MB"] = {
                "algo": algo, "ms": round(ms, 4), "busbw_gbs": round(bus, 1),
                "frac_of_link_900": round(bus / NVLINK_LINK_GBS, 4),
                "frac_of_measured_770": round(bus / NVLINK_GBS, 4),
                "nccl_ms": round(nccl_ms, 4),
                "nccl_busbw_gbs": round(factor * nbytes / (nccl_ms * 1e-3) / 1e9, 1),
            }
        ctx.check_status()

    if rank == 0:
        line = {
            "metric": "tp_mlp_fused_tflops (AG->GEMM + GEMM->RS; speedup vs NCCL+cuBLAS unfused; "
                      "% of roofline; all-reduce bus GB/s)",
            "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours",
            "config": {
                "model": "TP MLP block (hidden 8192, intermediate 28672), AG->GEMM + GEMM->RS",
                "global_batch": T, "seq_len": 1, "tokens": T, "hidden": H, "intermediate": I,
                "parallelism": f"tp{world}+sp{world}",
                "l2_policy": "inputs larger than L2: weights %.0f MB + activations %.0f MB per rank "
                             "per step" % (2 * H * I / world * 2 / 1e6,
                                           (T * H * 2 / world * 2 + T * I / world * 2) / 1e6),
            },
            "tokens_per_s": round(T / (ms_step * 1e-3), 1),
            "unfused_ms_per_step": round(base_ms, 4),
            "speedup_vs_unfused": round(base_ms / ms_step, 4),
            "roofline": {
                "peaks": peaks, "nvlink_gbs": NVLINK_GBS, "nvlink_link_gbs": NVLINK_LINK_GBS,
                "frac_of_sustained_at_link_rate": round(
                    roof(peaks["bf16_tflops_sustained"], NVLINK_LINK_GBS) / ms_step, 4),
                "target_ms_burst": round(roof(peaks["bf16_tflops"]), 4),
                "target_ms_sustained": round(roof(peaks["bf16_tflops_sustained"]), 4),
                "frac_of_burst": round(roof(peaks["bf16_tflops"]) / ms_step, 4),
                "frac_of_sustained": round(roof(peaks["bf16_tflops_sustained"]) / ms_step, 4),
                "note": "of %s" % peaks["source"],
            },
            "max_rel_err_vs_unfused": rel,
            "clocks": clocks,
            "e2e": {
                "value": round(flops / (e2e_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "ms_per_step": round(e2e_ms, 4),
                "unfused_ms_per_step": round(e2e_base_ms, 4),
                "h2d_bytes_per_step": Tl * H * 2, "d2h_bytes_per_step": 4,
            },
            "gpu_launches": mlp.launches_per_step * args.steps,
            "symmetric_memory": {"mode": ctx.mode, "multicast": ctx.has_multicast},
            **extras,
        }
        print(json.dumps(line), flush=True)
    sync_all()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
