"""Result store and summary writer.

Results are appended to a JSONL file keyed by a hash of (op, variant, shape, dtype, world), so
an interrupted sweep resumes by skipping finished keys; ``write_summary`` turns the store into
one ``summary.json`` (+ CSV) with, per entry, correctness, device time (max over ranks),
baseline time, speed-up, bytes / FLOPs, fraction of roofline and the verdict.  The JSON layout
keeps the reference's ``summary.json`` ideas (``metrics_comparison``, ``performance``,
``performance_detail``: datasets/readme.md:259-295, datasets/summary_template.json).
"""
from __future__ import annotations

import csv
import hashlib
import json
import os
import time

from . import registry, verdict


def config_key(op: str, variant: str, shape, dtype: str, world: int) -> str:
    blob = json.dumps([op, variant, list(shape) if not isinstance(shape, dict) else shape, dtype,
                       world], sort_keys=True)
    return hashlib.sha256(blob.encode()).hexdigest()[:16]


class ResultStore:
    def __init__(self, path: str):
        self.path = path
        self.done: dict[str, dict] = {}
        if os.path.exists(path):
            with open(path) as f:
                for line in f:
                    line = line.strip()
                    if line:
                        try:
                            r = json.loads(line)
                            self.done[r["key"]] = r
                        except Exception:
                            continue   # a torn last line of an interrupted run

    def has(self, key: str) -> bool:
        return key in self.done

    def add(self, rec: dict):
        rec = dict(rec)
        rec.setdefault("ts", time.time())
        self.done[rec["key"]] = rec
        os.makedirs(os.path.dirname(os.path.abspath(self.path)) or ".", exist_ok=True)
        with open(self.path, "a") as f:
            f.write(json.dumps(rec) + "\n")

    def records(self) -> list[dict]:
        """Measurements only (suite markers are book-keeping)."""
        return [r for r in self.done.values() if not str(r.get("op", "")).startswith("_")]


class SuiteLedger:
    """Suite-level resume for a multi-rank sweep.

    A suite is collective code: either every rank runs it or none does.  Each rank appends a
    marker record when it has finished a suite; on a resumed run a suite is skipped only when
    EVERY rank holds its marker (``agree`` reduces a bool with AND over the ranks), so ranks whose
    files diverged after an interrupted run still take the same branch.  The marker key covers
    the arguments that change what a suite measures."""

    def __init__(self, store: ResultStore, world: int, params: dict, agree=None, enabled: bool = True):
        self.store, self.world, self.enabled = store, world, enabled
        self.params = json.dumps(params, sort_keys=True)
        self.agree = agree or (lambda flag: flag)

    def _key(self, suite: str) -> str:
        return config_key("_suite", suite, {"params": self.params}, "-", self.world)

    def done(self, suite: str) -> bool:
        mine = self.enabled and self.store.has(self._key(suite))
        return bool(self.agree(bool(mine)))

    def mark(self, suite: str):
        self.store.add({"key": self._key(suite), "op": "_suite", "variant": suite, "world": self.world})


def finish_record(rec: dict) -> dict:
    """Adds speed-up and verdict to a raw measurement record."""
    out = dict(rec)
    base, ours = rec.get("baseline_ms"), rec.get("time_ms")
    if base and ours:
        out["speedup"] = base / ours
    v = verdict.compute_verdict(registry.entry(rec["op"]),
                                {"time_ms": base} if base else {},
                                {"time_ms": ours} if ours is not None else {})
    out["verdict"] = v.verdict
    out["performance_detail"] = v.detail
    return out


def export_performance_reference(rows: list[dict], out_dir: str, meta: dict | None = None) -> list[str]:
    """One JSON file per (op, variant, world) with the measured points over sizes, in the shape
    programs of the task harness print (``metrics: [{data_size, latency_avg, throughput_avg}]``):
    the stored numbers later runs are compared against - the role of the reference's
    ``datasets/performance_reference/*.json``."""
    os.makedirs(out_dir, exist_ok=True)
    groups: dict[tuple, list[dict]] = {}
    for r in rows:
        if r.get("time_ms") is None:
            continue
        groups.setdefault((r["op"], r.get("variant", ""), r.get("world", 1)), []).append(r)
    written = []
    for (op, variant, world), rs in sorted(groups.items()):
        pts = []
        for r in sorted(rs, key=lambda x: x.get("bytes") or _numel(x.get("shape"))):
            thr = r.get("busbw_gbs") if r.get("busbw_gbs") is not None else r.get("tflops")
            pts.append({"data_size": _numel(r.get("shape")), "shape": r.get("shape"),
                        "latency_avg": r["time_ms"] * 1e3, "throughput_avg": thr,
                        "baseline_latency_avg": (r["baseline_ms"] * 1e3) if r.get("baseline_ms") else None,
                        "roofline_frac": r.get("roofline_frac"), "verdict": r.get("verdict")})
        doc = {"op": op, "variant": variant, "world": world, "dtype": rs[0].get("dtype"),
               "Correctness": "PASS" if all(r.get("correct", True) for r in rs) else "FAIL",
               "data_size_unit": "elements", "latency_unit": "us",
               "throughput_unit": "GB/s (bus)" if rs[0].get("busbw_gbs") is not None else "TFLOP/s",
               "hardware": (meta or {}).get("hardware", "8x NVIDIA B200 (NVLink 5 / NVSwitch)"),
               "metrics": pts}
        path = os.path.join(out_dir, f"{op}_{variant or 'default'}_w{world}.json".replace("/", "-"))
        with open(path, "w") as f:
            json.dump(doc, f, indent=1)
        written.append(path)
    return written


def _numel(shape) -> int:
    n = 1
    for s in shape or []:
        n *= int(s)
    return n


def write_summary(records: list[dict], out_dir: str, meta: dict | None = None) -> dict:
    os.makedirs(out_dir, exist_ok=True)
    rows = [finish_record(r) for r in records]
    pairs = [(r["baseline_ms"], r["time_ms"]) for r in rows
             if r.get("baseline_ms") and r.get("time_ms") and r.get("correct", True)]
    summary = {
        "meta": meta or {},
        "verdict_scheme": {"better_pct": verdict.BETTER_PCT, "on_par_lower_pct": verdict.ON_PAR_LOWER_PCT,
                           "degraded_lower_pct": verdict.DEGRADED_LOWER_PCT},
        "counts": {v: sum(1 for r in rows if r["verdict"] == v) for v in verdict.ALL_VERDICTS},
        "all_correct": all(r.get("correct", True) for r in rows),
        "geomean_speedup": verdict.geometric_mean_speedup(pairs) if pairs else None,
        "entries": rows,
    }
    with open(os.path.join(out_dir, "summary.json"), "w") as f:
        json.dump(summary, f, indent=1)
    export_performance_reference(rows, os.path.join(out_dir, "performance_reference"), meta)
    cols = ["op", "variant", "world", "dtype", "shape", "correct", "max_err", "time_ms",
            "baseline_ms", "speedup", "busbw_gbs", "tflops", "roofline_frac", "verdict"]
    with open(os.path.join(out_dir, "summary.csv"), "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(cols)
        for r in rows:
            w.writerow([json.dumps(r.get(c)) if isinstance(r.get(c), (list, dict)) else r.get(c)
                        for c in cols])
    return summary
