"""Build / run / compare one source file of a task from the command line.

    python -m commbench_b200.harness.task_runner --task T --source FILE [--output BIN]
        [--build-only | --run-only] [--results-dir D] [--plot]
    python -m commbench_b200.harness.task_runner --task T --compare REF GEN --results-dir D

Functions ``build()``, ``run()``, ``build_and_run()`` and ``compare()`` are importable with the
same meaning.  ``compare`` builds and runs reference then candidate, writes per-size CSV files,
``summary.json`` (with the unified performance verdict) and, with ``--plot``, SVG line charts of
latency and throughput over message size (drawn without a plotting library).

One generic runner replaces the per-example ``build_and_run.py`` scripts of the reference
(canonical copy datasets/example001_gpu_comm_single_process/nv/build_and_run.py: result classes
:42-78, first-balanced-braces JSON extraction :103-122, ``build`` :125-217, ``run`` :220-262,
metric averages :305-317, CSV :320-328, plots :331-426, ``compare`` :488-693, CLI :696-868); the
launch recipe (plain, ``torchrun`` with W ranks, or an nvcc-built binary) comes from the task's
``task.json`` instead of being hard-coded per example.
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import sys

from . import compile_run as CR


def build(task_dir: str, source: str, output_dir: str | None = None) -> CR.CompileRunResult:
    return CR.compile_and_run(task_dir, source, build_only=True, work_dir=output_dir)


def run(task_dir: str, source: str, output_dir: str | None = None,
        timeout_s: float | None = None) -> CR.CompileRunResult:
    return CR.compile_and_run(task_dir, source, timeout_s, work_dir=output_dir)


build_and_run = run


def write_metrics_csv(result_json: dict | None, path: str) -> int:
    rows = (result_json or {}).get("metrics") or []
    cols = sorted({k for r in rows if isinstance(r, dict) for k in r})
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(cols)
        for r in rows:
            w.writerow([r.get(c) for c in cols])
    return len(rows)


def svg_line_chart(series: dict[str, list[tuple[float, float]]], title: str, xlabel: str,
                   ylabel: str, path: str, width: int = 720, height: int = 420) -> str:
    """Minimal log-x line chart as SVG text (no third-party plotting package needed)."""
    import math

    pts = [p for s in series.values() for p in s if p[0] > 0]
    if not pts:
        return ""
    x0, x1 = math.log2(min(p[0] for p in pts)), math.log2(max(p[0] for p in pts))
    y1 = max(p[1] for p in pts) or 1.0
    L, R, T, B = 70, 20, 40, 50
    sx = lambda x: L + (math.log2(x) - x0) / max(x1 - x0, 1e-9) * (width - L - R)
    sy = lambda y: height - B - y / y1 * (height - T - B)
    colors = ["#1f77b4", "#d62728", "#2ca02c", "#9467bd"]
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" '
           f'font-family="sans-serif" font-size="12">',
           f'<rect width="100%" height="100%" fill="white"/>',
           f'<text x="{width / 2}" y="20" text-anchor="middle" font-size="14">{title}</text>',
           f'<line x1="{L}" y1="{height - B}" x2="{width - R}" y2="{height - B}" stroke="black"/>',
           f'<line x1="{L}" y1="{T}" x2="{L}" y2="{height - B}" stroke="black"/>',
           f'<text x="{width / 2}" y="{height - 10}" text-anchor="middle">{xlabel} (log2)</text>',
           f'<text x="15" y="{height / 2}" transform="rotate(-90 15 {height / 2})" '
           f'text-anchor="middle">{ylabel}</text>',
           f'<text x="{L - 5}" y="{T + 4}" text-anchor="end">{y1:.3g}</text>',
           f'<text x="{L - 5}" y="{height - B}" text-anchor="end">0</text>']
    for i, (name, s) in enumerate(series.items()):
        s = sorted(p for p in s if p[0] > 0)
        if not s:
            continue
        d = " ".join(f"{'M' if j == 0 else 'L'}{sx(x):.1f},{sy(y):.1f}" for j, (x, y) in enumerate(s))
        c = colors[i % len(colors)]
        out.append(f'<path d="{d}" fill="none" stroke="{c}" stroke-width="2"/>')
        out += [f'<circle cx="{sx(x):.1f}" cy="{sy(y):.1f}" r="3" fill="{c}"/>' for x, y in s]
        out.append(f'<text x="{width - R - 150}" y="{T + 16 * (i + 1)}" fill="{c}">{name}</text>')
    out.append("</svg>")
    svg = "\n".join(out)
    with open(path, "w") as f:
        f.write(svg)
    return svg


def compare(task_dir: str, ref_source: str, gen_source: str, results_dir: str,
            plot: bool = False, timeout_s: float | None = None) -> dict:
    summary = CR.compare_save_results(task_dir, ref_source, gen_source, results_dir, timeout_s)
    # Per-size tables (and charts) from the programs' own "metrics" lists.
    runs = {}
    for tag in ("ref", "gen"):
        p = os.path.join(results_dir, f"{tag}_output.txt")
        j = None
        if os.path.exists(p):
            with open(p) as f:
                j = CR.first_json_object(f.read())
        runs[tag] = j
        write_metrics_csv(j, os.path.join(results_dir, f"{tag}_metrics.csv"))
    if plot:
        for key, label in (("latency_avg", "latency"), ("throughput_avg", "throughput")):
            series = {}
            for tag, name in (("ref", "reference"), ("gen", "generated")):
                rows = (runs[tag] or {}).get("metrics") or []
                series[name] = [(float(r["data_size"]), float(r[key])) for r in rows
                                if isinstance(r, dict) and "data_size" in r and key in r]
            unit = (runs["ref"] or runs["gen"] or {}).get(f"{label}_unit", "")
            svg_line_chart(series, f"{label} vs message size", "data size", f"{label} [{unit}]",
                           os.path.join(results_dir, f"{label}.svg"))
    return summary


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--task", required=True, help="task folder (or its name under harness/tasks)")
    ap.add_argument("--source")
    ap.add_argument("--output", default=None, help="build directory")
    ap.add_argument("--arch", default="sm_100a", help="accepted for compatibility; only sm_100a is built")
    ap.add_argument("--build-only", action="store_true")
    ap.add_argument("--run-only", action="store_true", help="alias of the default (build is cached by nvcc)")
    ap.add_argument("--compare", nargs=2, metavar=("REF", "GEN"))
    ap.add_argument("--results-dir", default="results")
    ap.add_argument("--plot", action="store_true")
    ap.add_argument("--timeout", type=float, default=None)
    a = ap.parse_args(argv)
    task = a.task if os.path.isdir(a.task) else os.path.join(os.path.dirname(__file__), "tasks", a.task)
    if a.arch != "sm_100a":
        print("only sm_100a is supported", file=sys.stderr)
        return 2
    if a.compare:
        s = compare(task, a.compare[0], a.compare[1], a.results_dir, a.plot, a.timeout)
        print(json.dumps({"performance": s["performance"], "correctness": s["correctness"]}))
        return 0 if s["correctness"]["generated"] else 1
    if not a.source:
        ap.error("--source or --compare is required")
    r = build(task, a.source, a.output) if a.build_only else run(task, a.source, a.output, a.timeout)
    if a.build_only:
        print("Build successful" if r.compile_success else r.compile_output)
        return 0 if r.compile_success else 1
    sys.stdout.write(r.run_stdout)
    sys.stderr.write(r.run_stderr)
    ok, why = CR.analyze_result(r)
    print(f"[task_runner] {why}", file=sys.stderr)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
