"""Roofline arithmetic of the harness: target time = the slower of (FLOPs / measured GEMM
peak) and (bytes that must cross NVLink per GPU and direction / measured link bandwidth).

Peaks come from ``MEASURED_PEAKS.json`` at the repository root when present (a STREAM-style
copy bandwidth and the cuBLAS bf16 throughput measured on the machines the numbers are taken
on), otherwise from the stated fall-back; every fraction is labelled with its source.  Bandwidth formulas follow the
reference's own conventions: ring-equivalent all-reduce bytes ``2(W-1)/W * S``
(datasets/example048_thunderkitten_all_reduce_easy/nv/empty_thunderkitten_all_reduce.cu:436,
datasets/example022_torch_distributed_nccl_allreduce/empty_nccl_allreduce.py:107-115), all-gather /
reduce-scatter ``(W-1)/W * S_total`` (datasets/example046_thunderkitten_all_gather_easy/nv/
empty_thunderkitten_all_gather.cu:504).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

NVLINK_GBS_MEASURED = 770.0   # peer copy, per direction per GPU (this pool)
NVLINK_GBS_NOMINAL = 900.0


@dataclass
class Peaks:
    bf16_tflops: float
    bf16_tflops_sustained: float
    hbm_gbs: float
    nvlink_gbs: float
    source: str


def load_peaks(root: str | None = None) -> Peaks:
    root = root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return Peaks(p["bf16_tflops"], p["bf16_tflops_sustained"], p["hbm_gbs"],
                     NVLINK_GBS_MEASURED, "measured")
    except Exception:
        return Peaks(1590.0, 1400.0, 6650.0, NVLINK_GBS_MEASURED, "fallback")


def allreduce_bus_factor(world: int) -> float:
    return 2.0 * (world - 1) / world if world > 1 else 1.0


def nvlink_bytes(op: str, nbytes: float, world: int, nvls: bool = False) -> float:
    """Bytes per GPU and direction that an op must move for a message of ``nbytes``
    (all-reduce / broadcast: message size; all-gather / reduce-scatter / all-to-all: the full
    gathered / scattered size)."""
    if world <= 1:
        return 0.0
    f = (world - 1) / world
    if op == "all_reduce":
        return nbytes if nvls else 2.0 * f * nbytes
    if op in ("all_gather", "reduce_scatter", "all_to_all"):
        return f * nbytes
    if op == "broadcast":
        return nbytes
    raise KeyError(op)


def roofline_ms(flops: float, link_bytes: float, peaks: Peaks, sustained: bool = False) -> float:
    tf = peaks.bf16_tflops_sustained if sustained else peaks.bf16_tflops
    t_compute = flops / (tf * 1e12) if flops else 0.0
    t_link = link_bytes / (peaks.nvlink_gbs * 1e9) if link_bytes else 0.0
    return max(t_compute, t_link) * 1e3


def fraction(target_ms: float, measured_ms: float) -> float | None:
    return None if not measured_ms else target_ms / measured_ms
