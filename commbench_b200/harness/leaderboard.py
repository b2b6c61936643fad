"""Batch evaluation over the shipped tasks and the model leaderboard.

    python -m commbench_b200.harness.leaderboard --run --model M [--tasks a,b,...] [--max-rounds R]
    python -m commbench_b200.harness.leaderboard --run --model reference --self-check
    python -m commbench_b200.harness.leaderboard [--out leaderboard.md]      # only aggregate

``--run`` drives :func:`eval_driver.generate_eval_one` over the tasks (those that need a GPU
are skipped on a machine without one), ``--self-check`` evaluates every task's own reference
solution as the candidate, which exercises the whole build / run / compare path without a model.
Aggregation reads ``tasks/<task>/results/<model>/summary.json`` and reports, per model, the
reference's leaderboard columns (README.md:71-79): pass rate, pass-and-good rate (correct AND
``better`` / ``on_par``), the geometric mean of candidate-over-reference speed-ups on the
correct tasks, and pass rate x geometric mean.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

from . import compile_run as CR
from . import eval_driver as ED

GOOD = {"better", "on_par"}


def has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:                                  # noqa: BLE001
        return False


def runnable_tasks(tasks_dir: str | None = None, names: list[str] | None = None) -> list[str]:
    root = tasks_dir or ED.TASKS_DIR
    gpu = has_gpu()
    out = []
    for t in sorted(os.listdir(root)):
        folder = os.path.join(root, t)
        if not os.path.exists(os.path.join(folder, "task.json")) or (names and t not in names):
            continue
        spec = CR.load_task(folder)
        if spec["needs_gpu"] and not gpu:
            continue
        out.append(t)
    return out


def run_all(model: str, tasks_dir: str | None = None, names: list[str] | None = None,
            max_rounds: int = 3, self_check: bool = False, generate=None, quiet: bool = True,
            log=print) -> list[dict]:
    rows = []
    root = tasks_dir or ED.TASKS_DIR
    for t in runnable_tasks(tasks_dir, names):
        cand = CR.find_ref_file(os.path.join(root, t)) if self_check else None
        passed, reason, _, rounds, perf = ED.generate_eval_one(
            t, model, max_rounds, tasks_dir=tasks_dir, save=False, quiet=quiet, generate=generate,
            candidate=cand)
        rows.append({"task": t, "passed": passed, "reason": reason, "rounds": rounds,
                     "performance": (perf or {}).get("performance")})
        log(json.dumps(rows[-1]))
    return rows


def speedup_of(summary: dict) -> float | None:
    """Candidate over reference on the task's primary metric (> 1 = candidate faster)."""
    d = summary.get("performance_detail") or {}
    ref, gen = d.get("baseline", d.get("ref")), d.get("candidate", d.get("generated"))
    if not ref or not gen or ref <= 0 or gen <= 0:
        return None
    return gen / ref if d.get("direction") == "higher" else ref / gen


def collect(tasks_dir: str | None = None) -> list[dict]:
    root = tasks_dir or ED.TASKS_DIR
    out = []
    for t in sorted(os.listdir(root)):
        rdir = os.path.join(root, t, "results")
        if not os.path.isdir(rdir):
            continue
        for model in sorted(os.listdir(rdir)):
            p = os.path.join(rdir, model, "summary.json")
            if os.path.exists(p):
                with open(p) as f:
                    s = json.load(f)
                s.setdefault("task", t)
                s.setdefault("model", model)
                out.append(s)
    return out


def score(summaries: list[dict]) -> dict[str, dict]:
    by_model: dict[str, list[dict]] = {}
    for s in summaries:
        by_model.setdefault(s["model"], []).append(s)
    table = {}
    for model, rows in by_model.items():
        n = len(rows)
        correct = [r for r in rows if r.get("pass_iteration") is not None]
        good = [r for r in correct if r.get("performance") in GOOD or r.get("performance") == "info_only"]
        sp = [x for x in (speedup_of(r) for r in correct) if x is not None]
        gm = math.exp(sum(math.log(x) for x in sp) / len(sp)) if sp else None
        rate = len(correct) / n if n else 0.0
        table[model] = {"tasks": n, "correct": len(correct), "pass_rate": rate,
                        "pass_good_rate": len(good) / n if n else 0.0, "gm_speedup": gm,
                        "pass_x_gm": rate * gm if gm is not None else None,
                        "mean_rounds_to_pass": (sum(r["pass_iteration"] for r in correct) / len(correct))
                        if correct else None}
    return table


def render_markdown(table: dict[str, dict]) -> str:
    fmt = lambda v, p="{:.2f}": "-" if v is None else p.format(v)
    lines = ["| model | tasks | pass rate | pass + good | GM speed-up | pass x GM | mean rounds to pass |",
             "|---|---|---|---|---|---|---|"]
    order = sorted(table, key=lambda m: (-(table[m]["pass_x_gm"] or 0.0), -table[m]["pass_rate"], m))
    for m in order:
        r = table[m]
        lines.append(f"| {m} | {r['tasks']} | {fmt(r['pass_rate'] * 100, '{:.0f} %')} | "
                     f"{fmt(r['pass_good_rate'] * 100, '{:.0f} %')} | {fmt(r['gm_speedup'])} | "
                     f"{fmt(r['pass_x_gm'])} | {fmt(r['mean_rounds_to_pass'], '{:.1f}')} |")
    return "\n".join(lines) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--run", action="store_true")
    ap.add_argument("--model", default="gpt-4o")
    ap.add_argument("--tasks", default=None, help="comma-separated task names (default: all runnable)")
    ap.add_argument("--tasks-dir", default=None)
    ap.add_argument("--max-rounds", type=int, default=3)
    ap.add_argument("--self-check", action="store_true")
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    if a.run:
        run_all(a.model, a.tasks_dir, a.tasks.split(",") if a.tasks else None, a.max_rounds,
                a.self_check)
    table = score(collect(a.tasks_dir))
    md = render_markdown(table)
    if a.out:
        with open(a.out, "w") as f:
            f.write(md)
        with open(os.path.splitext(a.out)[0] + ".json", "w") as f:
            json.dump(table, f, indent=1)
    print(md, end="")
    return 0


if __name__ == "__main__":
    sys.exit(main())
