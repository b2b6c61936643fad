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
    if key not in candidate_metrics or candidate_metrics[key] is None:
        return Verdict(NO_CANDIDATE_METRICS, {"primary_metric": key})
    if key not in baseline_metrics or baseline_metrics[key] is None:
        return Verdict(NO_BASELINE_METRICS, {"primary_metric": key})
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
