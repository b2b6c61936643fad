"""Generate -> build -> run -> compare -> repair, for one task.

    python -m commbench_b200.harness.eval_driver <task> --model M [--max-rounds R]
        [--temperature T] [--tasks-dir D] [--no-save] [--no-ref] [--quiet] [--list-models]
        [--candidate FILE]      # evaluate an existing file instead of asking a model

A round asks the model for the program (first round: completion prompt; later rounds: a fix
prompt carrying up to two earlier failed attempts as diffs, or a performance prompt carrying the
comparison summary), saves it as ``generated_<task>_<model>_round<N>_<stamp>.<ext>``, builds and
runs it under the execution lock, and - when a reference implementation exists - runs reference
and candidate back to back and takes the unified verdict.  The loop ends on an acceptable
verdict (``better`` / ``on_par`` / ``info_only``, or correctness alone without a reference) or
when the rounds run out.  Every round leaves ``prompt.txt`` and ``build_run_output.txt`` in
``results/<model>/round<N>_<stamp>/``; the final ``summary.json`` records the model and the
rounds at which the program first passed and last improved.

Counterpart of the reference's ``scripts/generate_eval_one.py`` (``generate_eval_one`` :120-651,
transient-error retry with ``base * 2^n + jitter`` back-off :52-117, CLI :654-819).
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import sys
import time

from . import compile_run as CR
from .llm import factory as F
from .llm import prompt as P
from .verdict import ACCEPTABLE    # one definition: the driver and the verdict module agree

TASKS_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tasks")


def _safe(name: str) -> str:
    return "".join(c if c.isalnum() or c in "-_." else "_" for c in name)


def call_with_retry(fn, attempts: int = 4, base: float = 2.0, sleep=time.sleep, log=None):
    """Runs ``fn`` again after transient failures (rate limits, time-outs, 5xx), waiting
    ``base * 2^n`` plus jitter in between; anything else is raised at once."""
    for n in range(attempts):
        try:
            return fn()
        except Exception as e:                     # noqa: BLE001
            if n == attempts - 1 or not F.is_transient(e):
                raise
            delay = F.backoff_delay(n, base)
            if log:
                log(f"transient model error ({e}); retry {n + 1} in {delay:.1f}s")
            sleep(delay)


def generate_eval_one(task: str, model: str = "gpt-4o", max_rounds: int = 3,
                      temperature: float | None = 0.2, tasks_dir: str | None = None,
                      save: bool = True, use_ref: bool = True, quiet: bool = False,
                      generate=None, execution_lock=None, timeout_s: float | None = 180,
                      candidate: str | None = None):
    """Returns ``(passed, reason, result, rounds, perf)``: ``result`` is the last
    ``CompileRunResult``, ``rounds`` the number of rounds used, ``perf`` the last comparison
    summary (or ``None``).  ``generate(prompt, model, language, temperature) -> code`` replaces
    the model call; ``execution_lock`` is any context manager that serialises GPU use between
    concurrent drivers."""
    say = (lambda *a: None) if quiet else (lambda *a: print(*a, flush=True))
    folder = os.path.join(tasks_dir or TASKS_DIR, task) if not os.path.isdir(task) else task
    skeleton = CR.find_empty_file(folder)
    if skeleton is None:
        return False, f"no skeleton (empty_*) in {folder}", None, 0, None
    ref = CR.find_ref_file(folder) if use_ref else None
    if ref is None:
        say("no reference implementation: correctness only")
    spec = CR.load_task(folder)
    lang = P.language_of(skeleton)
    ext = os.path.splitext(skeleton)[1]
    gen = generate or (lambda pr, mo, la, te: F.generate_code(pr, mo, la, te))
    lock = execution_lock if execution_lock is not None else contextlib.nullcontext()
    out_root = os.path.join(folder, "results", _safe(model))

    prompt = P.generate_completion_prompt(skeleton, spec.get("description"))
    history: list[dict] = []
    result, perf, reason = None, None, "no round ran"
    pass_round = improve_round = None
    for rnd in range(1, max_rounds + 1):
        stamp = time.strftime("%Y%m%d_%H%M%S")
        if candidate is not None:
            with open(candidate, encoding="utf-8") as f:
                code = f.read()
        else:
            say(f"[round {rnd}] asking {model}")
            code = call_with_retry(lambda: gen(prompt, model, lang, temperature), log=say)
        rdir = os.path.join(out_root, f"round{rnd}_{stamp}")
        gen_path = os.path.join(folder if save else rdir,
                                f"generated_{spec['name']}_{_safe(model)}_round{rnd}_{stamp}{ext}")
        os.makedirs(os.path.dirname(gen_path), exist_ok=True)
        os.makedirs(rdir, exist_ok=True)
        with open(gen_path, "w", encoding="utf-8") as f:
            f.write(code)
        P.save_prompt_to_file(prompt, os.path.join(rdir, "prompt.txt"))
        with lock:
            result = CR.compile_and_run(folder, gen_path, timeout_s, work_dir=os.path.join(rdir, "build"))
        with open(os.path.join(rdir, "build_run_output.txt"), "w", encoding="utf-8") as f:
            f.write(result.output)
        ok, reason = CR.analyze_result(result)
        say(f"[round {rnd}] {'ok' if ok else 'FAILED'}: {reason}")
        if not ok:
            err = CR.get_error_details(result)
            prompt = P.generate_fix_prompt_from_code(skeleton, code, err, history)
            history.append({"code": code, "error": err})
            if candidate is not None:
                break
            continue
        if pass_round is None:
            pass_round = rnd
        if ref is None:
            improve_round = rnd
            break
        with lock:
            perf = CR.compare_save_results(folder, ref, gen_path, rdir, timeout_s)
        verdict = perf.get("performance")
        say(f"[round {rnd}] verdict vs reference: {verdict}")
        improve_round = rnd
        if verdict in ACCEPTABLE or candidate is not None:
            break
        reason = f"performance verdict {verdict}"
        prompt = P.generate_perf_fix_prompt_from_code(skeleton, code, perf)
    passed = pass_round is not None and (perf is None or perf.get("performance") in ACCEPTABLE
                                         or ref is None)
    rounds = rnd if max_rounds > 0 else 0
    final = {"task": spec["name"], "model": model, "passed": passed, "reason": reason,
             "rounds": rounds, "pass_iteration": pass_round, "improvement_iteration": improve_round,
             "performance": (perf or {}).get("performance"),
             "performance_detail": (perf or {}).get("performance_detail"),
             "metrics_comparison": (perf or {}).get("metrics_comparison")}
    os.makedirs(out_root, exist_ok=True)
    with open(os.path.join(out_root, "summary.json"), "w") as f:
        json.dump(final, f, indent=1)
    return passed, reason, result, rounds, perf


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("task", nargs="?")
    ap.add_argument("--model", default="gpt-4o")
    ap.add_argument("--max-rounds", type=int, default=3)
    ap.add_argument("--temperature", type=float, default=0.2)
    ap.add_argument("--tasks-dir", default=None)
    ap.add_argument("--no-save", action="store_true", help="keep generated files under results/ only")
    ap.add_argument("--no-ref", action="store_true", help="correctness only")
    ap.add_argument("--quiet", action="store_true")
    ap.add_argument("--candidate", default=None, help="evaluate this file instead of calling a model")
    ap.add_argument("--list-models", action="store_true")
    ap.add_argument("--list-tasks", action="store_true")
    a = ap.parse_args(argv)
    if a.list_models:
        print(json.dumps(F.list_supported_models(), indent=1))
        return 0
    root = a.tasks_dir or TASKS_DIR
    if a.list_tasks or not a.task:
        for t in sorted(os.listdir(root)):
            if os.path.isdir(os.path.join(root, t)):
                print(t)
        return 0
    passed, reason, _, rounds, perf = generate_eval_one(
        a.task, a.model, a.max_rounds, a.temperature, a.tasks_dir, not a.no_save, not a.no_ref,
        a.quiet, candidate=a.candidate)
    print(json.dumps({"task": a.task, "passed": passed, "reason": reason, "rounds": rounds,
                      "performance": (perf or {}).get("performance")}))
    return 0 if passed else 1


if __name__ == "__main__":
    sys.exit(main())
