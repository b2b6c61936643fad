"""Prompts for the generate -> build -> run -> repair loop, and extraction of code from replies.

Prompt kinds: *completion* (fill in the skeleton of a task; a *detailed* variant adds the
machine and hints), *fix* (the last attempt failed to build / run / verify: show earlier attempts
as capped diffs plus capped error text), *performance fix* (it works but the verdict against the
reference is below par: show the comparison summary), *optimisation* (make a working program
faster, with or without its measured metrics) and *explanation* (describe what a source file
does).

Counterpart of the reference's ``prompt_llm/prompt.py``: completion prompt with C++/CUDA and
Python variants (:167-247), code extraction from fenced or truncated replies (:104-164), fix
prompt with numbered earlier rounds as capped unified diffs and capped errors (:18-19, :33-52,
:353-470), performance-fix prompt embedding ``summary.json`` (:473-534).  The wording here is
written for this framework's targets: one architecture (sm_100a), bounded waits, one JSON line
of results.
"""
from __future__ import annotations

import difflib
import json
import os
import re

MAX_DIFF_CHARS = 3000
MAX_ERROR_CHARS = 1500
MAX_HISTORY = 2

_LANG = {".py": "python", ".cu": "cuda", ".cuh": "cuda", ".cpp": "cpp", ".cc": "cpp", ".cxx": "cpp",
         ".h": "cpp"}

_RULES_NATIVE = """Rules:
- Target one GPU architecture: NVIDIA B200 (sm_100a).  Do not add code paths for other vendors.
- Keep every public name, signature, command-line flag and the printed JSON schema of the skeleton.
- Every wait on a flag, peer or mbarrier must be bounded (iteration or time limit) and must report
  failure through a status value; never spin forever, never trap.
- Do not start TMA loads with cluster multicast from memory that another GPU owns.
- The program prints exactly one JSON object with the results; "Correctness" is "PASS" or "FAIL".
- Reply with the complete source file in one fenced code block and nothing else."""

_RULES_PYTHON = """Rules:
- Keep every public name, signature, command-line flag and the printed JSON schema of the skeleton.
- One process per GPU; rendezvous on 127.0.0.1; no network access, no extra packages.
- Time on the device (CUDA events), after warm-up, maximum over ranks.
- The program prints exactly one JSON object with the results; "Correctness" is "PASS" or "FAIL".
- Reply with the complete source file in one fenced code block and nothing else."""


def language_of(path: str) -> str:
    return _LANG.get(os.path.splitext(path)[1].lower(), "text")


def _read(path: str) -> str:
    with open(path, encoding="utf-8", errors="replace") as f:
        return f.read()


def _cap(text: str, limit: int, keep_tail: bool = True) -> str:
    text = text.strip()
    if len(text) <= limit:
        return text
    cut = len(text) - limit
    return (f"[... {cut} characters omitted ...]\n" + text[-limit:]) if keep_tail else \
        (text[:limit] + f"\n[... {cut} characters omitted ...]")


def generate_completion_prompt(skeleton_path: str, task_description: str | None = None) -> str:
    code = _read(skeleton_path)
    lang = language_of(skeleton_path)
    rules = _RULES_PYTHON if lang == "python" else _RULES_NATIVE
    what = task_description or "Complete every part marked TODO so that the program builds, runs and verifies."
    return (f"You are completing a GPU communication benchmark program ({lang}).\n\n{what}\n\n{rules}\n\n"
            f"Skeleton ({os.path.basename(skeleton_path)}):\n```{lang}\n{code}\n```\n")


def render_diff(before: str, after: str, name: str = "source", limit: int = MAX_DIFF_CHARS) -> str:
    diff = "".join(difflib.unified_diff(before.splitlines(True), after.splitlines(True),
                                        fromfile=f"{name} (skeleton)", tofile=f"{name} (attempt)",
                                        n=2))
    return _cap(diff, limit, keep_tail=False) if diff else "(no textual change)"


def generate_fix_prompt_from_code(skeleton_path: str, current_code: str, error_text: str,
                                  history: list[dict] | None = None) -> str:
    """``history`` = earlier failed attempts, oldest first: ``{"code": ..., "error": ...}``.
    Only the last ``MAX_HISTORY`` are shown, as diffs against the skeleton."""
    skeleton = _read(skeleton_path)
    lang = language_of(skeleton_path)
    name = os.path.basename(skeleton_path)
    parts = [f"The program below ({lang}) failed. Fix it.\n",
             _RULES_PYTHON if lang == "python" else _RULES_NATIVE, ""]
    shown = (history or [])[-MAX_HISTORY:]
    first_no = len(history or []) - len(shown) + 1
    for i, h in enumerate(shown):
        parts.append(f"### Earlier attempt {first_no + i} (did not work either)\n"
                     f"```diff\n{render_diff(skeleton, h.get('code', ''), name)}\n```\n"
                     f"Its error:\n```\n{_cap(h.get('error', ''), MAX_ERROR_CHARS)}\n```\n")
    parts.append(f"### Current attempt\n```{lang}\n{current_code}\n```\n")
    parts.append(f"### Error of the current attempt\n```\n{_cap(error_text, MAX_ERROR_CHARS)}\n```\n")
    parts.append("Do not repeat the earlier attempts. Reply with the complete corrected file.")
    return "\n".join(parts)


def generate_perf_fix_prompt_from_code(skeleton_path: str, current_code: str, summary: dict | str) -> str:
    lang = language_of(skeleton_path)
    if not isinstance(summary, str):
        summary = json.dumps(summary, indent=1)
    return (f"The program below ({lang}) is correct but slower than the reference implementation.\n\n"
            f"Comparison (reference vs generated):\n```json\n{_cap(summary, 4000, keep_tail=False)}\n```\n\n"
            "Make it faster without changing what it computes or prints: fewer launches and host "
            "synchronisations, wider memory operations, overlap of copies with compute, fewer "
            "barriers, peer stores instead of staged copies.\n\n"
            f"{_RULES_PYTHON if lang == 'python' else _RULES_NATIVE}\n\n"
            f"Current program:\n```{lang}\n{current_code}\n```\n")


def generate_completion_prompt_detailed(skeleton_path: str, task_description: str | None = None,
                                        hardware: dict | None = None, hints: list[str] | None = None) -> str:
    """Completion prompt with the machine it will run on and optional hints spelled out
    (the reference keeps such a variant beside the plain one: prompt_llm/prompt.py, "detailed")."""
    hw = hardware or {"gpu": "NVIDIA B200 (sm_100a), 148 SMs, 180 GB HBM3e", "gpus_per_node": 8,
                      "interconnect": "NVLink 5 through NVSwitch, 900 GB/s per direction per GPU, "
                                      "in-switch reduction (multimem) available"}
    lines = [generate_completion_prompt(skeleton_path, task_description).rstrip("\n"), "",
             "Machine:"] + [f"- {k}: {v}" for k, v in hw.items()]
    if hints:
        lines += ["", "Hints:"] + [f"- {h}" for h in hints]
    return "\n".join(lines) + "\n"


def generate_optimization_prompt(source_path: str, goal: str = "lower latency at every size") -> str:
    """Asks for a faster version of a working program without a measured comparison at hand."""
    lang = language_of(source_path)
    return (f"The {lang} program below works. Rewrite it for {goal} on one NVIDIA B200 node without changing "
            "what it computes, checks or prints.\n\n"
            f"{_RULES_PYTHON if lang == 'python' else _RULES_NATIVE}\n\n"
            f"Program ({os.path.basename(source_path)}):\n```{lang}\n{_read(source_path)}\n```\n")


def generate_performance_optimization_prompt(source_path: str, metrics: dict,
                                             roofline: dict | None = None) -> str:
    """Optimisation prompt that carries the program's own measured metrics and, when known, how far
    they are from the machine's limits (fraction of link bandwidth or of the GEMM peak)."""
    lang = language_of(source_path)
    text = (f"The {lang} program below works. Its measured results:\n```json\n"
            f"{_cap(json.dumps(metrics, indent=1), 3000, keep_tail=False)}\n```\n")
    if roofline:
        text += ("Against the machine's limits:\n```json\n"
                 f"{_cap(json.dumps(roofline, indent=1), 1500, keep_tail=False)}\n```\n")
    text += ("\nName the bottleneck these numbers point to (launch latency, synchronisation, link bandwidth, "
             "memory bandwidth, tensor throughput), then rewrite the program to remove it without changing what "
             "it computes, checks or prints.\n\n"
             f"{_RULES_PYTHON if lang == 'python' else _RULES_NATIVE}\n\n"
             f"Program ({os.path.basename(source_path)}):\n```{lang}\n{_read(source_path)}\n```\n")
    return text


def generate_explanation_prompt(source_path: str) -> str:
    lang = language_of(source_path)
    return (f"Explain what this {lang} program measures, how ranks synchronise and where its time goes. "
            f"Be specific and brief.\n```{lang}\n{_read(source_path)}\n```\n")


_FENCE = re.compile(r"```[ \t]*([A-Za-z0-9_+\-]*)[ \t]*\n(.*?)```", re.S)


def extract_code_from_response(reply: str, language: str | None = None) -> str:
    """The program in a model's reply: the largest fenced block (preferring a matching language
    tag); an unterminated fence (cut-off reply) yields everything after it; no fence at all
    yields the reply itself."""
    if not reply:
        return ""
    blocks = _FENCE.findall(reply)
    if blocks:
        want = (language or "").lower()
        alias = {"cuda": {"cuda", "cu", "cpp", "c++", "c"}, "cpp": {"cpp", "c++", "c", "cuda", "cu"},
                 "python": {"python", "py"}}.get(want, {want} if want else set())
        tagged = [b for t, b in blocks if t.lower() in alias]
        pool = tagged or [b for _, b in blocks]
        return max(pool, key=len).strip("\n") + "\n"
    m = re.search(r"```[ \t]*[A-Za-z0-9_+\-]*[ \t]*\n", reply)
    if m:                                   # opening fence without a closing one
        return reply[m.end():].rstrip("`\n ") + "\n"
    return reply.strip("\n") + "\n"


def save_prompt_to_file(prompt: str, path: str) -> str:
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    with open(path, "w", encoding="utf-8") as f:
        f.write(prompt)
    return path
