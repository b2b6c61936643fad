"""Performance verdicts: candidate (ours) against a baseline (NCCL + cuBLAS, unfused).

Same tiers and thresholds as the reference's unified verdict
(run_eval/perf_verdict.py:47-49 thresholds, :60-63 non-comparison verdicts, :272-295
did-not-measure guard, :298-306 classification, :309-397 verdict computation), applied to
"ours vs baseline on the same box" instead of "generated vs reference program".
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

BETTER_PCT = 20.0
ON_PAR_LOWER_PCT = -5.0
DEGRADED_LOWER_PCT = -40.0

BETTER = "better"
ON_PAR = "on_par"
DEGRADED = "degraded"
SEVERELY_DEGRADED = "severely_degraded"
INFO_ONLY = "info_only"
NO_CANDIDATE_METRICS = "no_candidate_metrics"
NO_BASELINE_METRICS = "no_baseline_metrics"
UNKNOWN = "unknown"

ALL_VERDICTS = (BETTER, ON_PAR, DEGRADED, SEVERELY_DEGRADED, INFO_ONLY, NO_CANDIDATE_METRICS,
                NO_BASELINE_METRICS, UNKNOWN)
# Verdicts after which no further tuning round is asked for.
ACCEPTABLE = frozenset({BETTER, ON_PAR, INFO_ONLY, NO_CANDIDATE_METRICS, NO_BASELINE_METRICS,
                        UNKNOWN})


def improvement_pct(baseline: float, candidate: float, direction: str):
    """(improvement %, note).  A time-like metric that reads 0 while the baseline is positive
    was not measured: it is pinned to -100 % instead of the naive +100 %."""
    if direction not in ("higher", "lower"):
        raise ValueError(f"direction must be 'higher' or 'lower', got {direction!r}")
    if direction == "lower" and baseline > 0 and candidate == 0:
        return -100.0, "candidate=0 with baseline>0 treated as did-not-measure"
    if baseline == 0:
        return 0.0, "baseline=0; treated as no-op"
    if direction == "lower":
        return (baseline - candidate) / baseline * 100.0, None
    return (candidate - baseline) / baseline * 100.0, None


def classify(pct: float) -> str:
    if pct >= BETTER_PCT:
        return BETTER
    if pct >= ON_PAR_LOWER_PCT:
        return ON_PAR
    if pct >= DEGRADED_LOWER_PCT:
        return DEGRADED
    return SEVERELY_DEGRADED


@dataclass
class Verdict:
    verdict: str
    detail: dict[str, Any] = field(default_factory=dict)

    @property
    def acceptable(self) -> bool:
        return self.verdict in ACCEPTABLE


def compute_verdict(entry, baseline_metrics: dict, candidate_metrics: dict) -> Verdict:
    """`entry` is a registry entry: "info_only", None (unknown op) or
    {"primary": key, "direction": "higher"|"lower"}."""
    if entry is None:
        return Verdict(UNKNOWN, {"note": "op missing from the metric registry"})
    if entry == "info_only":
        return Verdict(INFO_ONLY, {"note": "op has no numeric performance metric"})
    key, direction = entry["primary"], entry["direction"]

    def numeric(v) -> bool:
        return isinstance(v, (int, float)) and not isinstance(v, bool)

    # Candidate first; a value that is not a number ("N/A", a dict) counts as missing.
    if not numeric(candidate_metrics.get(key)):
        return Verdict(NO_CANDIDATE_METRICS, {"primary_metric": key})
    if not numeric(baseline_metrics.get(key)):
        return Verdict(NO_BASELINE_METRICS, {"primary_metric": key})
    if direction not in ("higher", "lower"):
        return Verdict(UNKNOWN, {"primary_metric": key, "note": f"bad direction {direction!r}"})
    b, c = float(baseline_metrics[key]), float(candidate_metrics[key])
    pct, note = improvement_pct(b, c, direction)
    d = {"primary_metric": key, "direction": direction, "baseline": b, "candidate": c,
         "improvement_pct": round(pct, 3)}
    if note:
        d["note"] = note
    return Verdict(classify(pct), d)


def geometric_mean_speedup(pairs) -> float:
    """GM over sizes of candidate/baseline speed-ups (the leaderboard's GM-speedup, README.md:71-79).
    `pairs` = iterable of (baseline_time, candidate_time)."""
    import math

    logs = [math.log(b / c) for b, c in pairs if b > 0 and c > 0]
    return math.exp(sum(logs) / len(logs)) if logs else float("nan")


def infer_task_name(path: str) -> str | None:
    """Name of the task a file or results folder belongs to: the nearest ancestor folder that
    holds a ``task.json`` (the reference walks up to ``exampleNNN_*``:
    run_eval/perf_verdict.py:256-269)."""
    import os

    d = os.path.abspath(path)
    if not os.path.isdir(d):
        d = os.path.dirname(d)
    while True:
        if os.path.exists(os.path.join(d, "task.json")):
            return os.path.basename(d)
        parent = os.path.dirname(d)
        if parent == d:
            return None
        d = parent


def override_summary_verdict(summary_path: str, entry=None) -> dict:
    """Re-judges a comparison ``summary.json`` written by an older or foreign tool with the
    unified scheme: recomputes ``performance`` / ``performance_detail`` from its
    ``metrics_comparison`` (either ``{metric: {reference, generated}}`` or the reference's
    ``{ref: {...}, generated: {...}}`` layout), keeps what was there as ``performance_legacy`` and
    records the thresholds used.  ``entry`` = ``{"primary", "direction"}`` or ``"info_only"``;
    by default the task's own ``task.json`` decides
    (run_eval/perf_verdict.py:400-452)."""
    import json
    import os

    with open(summary_path) as f:
        s = json.load(f)
    if entry is None:
        d = os.path.dirname(os.path.abspath(summary_path))
        spec = None
        while True:
            p = os.path.join(d, "task.json")
            if os.path.exists(p):
                with open(p) as f:
                    spec = json.load(f)
                break
            if os.path.dirname(d) == d:
                break
            d = os.path.dirname(d)
        entry = {"primary": spec["primary_metric"], "direction": spec.get("direction", "lower")} \
            if spec and spec.get("primary_metric") else INFO_ONLY
    mc = s.get("metrics_comparison") or {}
    if "ref" in mc and "generated" in mc and isinstance(mc["ref"], dict):
        base, cand = mc["ref"], mc["generated"]
    else:
        base = {k: v.get("reference") for k, v in mc.items() if isinstance(v, dict)}
        cand = {k: v.get("generated") for k, v in mc.items() if isinstance(v, dict)}
    v = compute_verdict(entry, {k: x for k, x in base.items() if x is not None},
                        {k: x for k, x in cand.items() if x is not None})
    if "performance" in s and "performance_legacy" not in s:
        s["performance_legacy"] = s["performance"]
    s["performance"], s["performance_detail"] = v.verdict, v.detail
    s["verdict_scheme"] = {"better_pct": BETTER_PCT, "on_par_lower_pct": ON_PAR_LOWER_PCT,
                           "degraded_lower_pct": DEGRADED_LOWER_PCT}
    with open(summary_path, "w") as f:
        json.dump(s, f, indent=1)
    return s
