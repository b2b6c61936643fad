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
        return list(self.done.values())


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
    cols = ["op", "variant", "world", "dtype", "shape", "correct", "max_err", "time_ms",
            "baseline_ms", "speedup", "busbw_gbs", "tflops", "roofline_frac", "verdict"]
    with open(os.path.join(out_dir, "summary.csv"), "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(cols)
        for r in rows:
            w.writerow([json.dumps(r.get(c)) if isinstance(r.get(c), (list, dict)) else r.get(c)
                        for c in cols])
    return summary
