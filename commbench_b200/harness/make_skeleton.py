"""Derives a task's ``empty_*`` skeleton from its ``ref_*`` solution.

A reference marks what the candidate has to write:

    # --- solution: what to do here
    #     (more lines of the same instruction)
    <code>
    # --- end solution

(``//`` instead of ``#`` in C++ / CUDA sources).  The skeleton keeps everything outside the
marked regions - the harness part of the program: inputs, checks, timing, the JSON line - and
replaces each region by a ``TODO`` comment with the instruction, followed by
``raise NotImplementedError`` in Python or nothing in C++ (a region may give a C++ fallback
statement after ``else:`` on the marker line, e.g. ``// --- solution else: return false;``).
A paragraph that starts with ``Reference counterpart:`` (where the exercise comes from) stays in
the solution only; other lines can be dropped with ``--drop-line-containing``.

    python -m commbench_b200.harness.make_skeleton tasks/x/ref_x.py [--check]

``--check`` compares with the committed skeleton instead of writing it (exit code 1 when they
differ), which is what the tests run.  The reference's data set keeps both files by hand
(datasets/readme.md:401-417: "the template keeps the harness so only TODO regions change").
"""
from __future__ import annotations

import argparse
import os
import re
import sys

_OPEN = re.compile(r"^(?P<ind>\s*)(?P<c>#|//) --- solution(?: else: (?P<else>.*?))?(?::\s*(?P<todo>.*))?$")
_CLOSE = re.compile(r"^\s*(#|//) --- end solution\s*$")


def skeleton_text(ref_text: str, drop_containing: tuple[str, ...] = ()) -> str:
    out, lines, i = [], ref_text.splitlines(), 0
    while i < len(lines):
        line = lines[i]
        m = _OPEN.match(line)
        if not m:
            if _CLOSE.match(line):
                raise ValueError(f"line {i + 1}: end marker without a solution marker")
            if line.strip().lstrip("/# ").startswith("Reference counterpart:"):
                # the paragraph that says where the exercise comes from stays in the solution only
                tok = next((t for t in ("//", "#") if line.strip().startswith(t)), None)
                while i < len(lines) and lines[i].strip() not in ("", "//", "#") \
                        and not lines[i].strip().startswith('"""') \
                        and (tok is None or lines[i].strip().startswith(tok + " ")):
                    i += 1                      # a comment paragraph ends where the comment ends
                if out and out[-1].strip() in ("", "//", "#") and i < len(lines) \
                        and lines[i].strip() in ("", "//", "#"):
                    i += 1                      # do not leave two blank lines behind
                elif out and out[-1].strip() == "" and i < len(lines) \
                        and lines[i].strip().startswith('"""'):
                    out.pop()                   # nor a blank line before the closing quotes
                elif tok and out and out[-1].strip() == tok and \
                        (i == len(lines) or not lines[i].strip().startswith(tok)):
                    out.pop()                   # nor an empty comment line at the end of the block
                continue
            if not any(d in line for d in drop_containing):
                out.append(line)
            i += 1
            continue
        ind, c = m.group("ind"), m.group("c")
        todo = [m.group("todo") or "implement"]
        i += 1
        cont = re.compile(r"^\s*" + re.escape(c) + r"     (.*)$")
        while i < len(lines) and cont.match(lines[i]) and not _CLOSE.match(lines[i]):
            todo.append(cont.match(lines[i]).group(1))
            i += 1
        while i < len(lines) and not _CLOSE.match(lines[i]):
            if _OPEN.match(lines[i]):
                raise ValueError(f"line {i + 1}: nested solution marker")
            i += 1
        if i == len(lines):
            raise ValueError("solution marker without an end marker")
        i += 1
        out.append(f"{ind}{c} TODO: {todo[0]}")
        out += [f"{ind}{c}       {t}" for t in todo[1:]]
        if c == "#":
            out.append(f"{ind}raise NotImplementedError")
        elif m.group("else"):
            out.append(f"{ind}{m.group('else')}")
    return "\n".join(out) + "\n"


def skeleton_path(ref_path: str) -> str:
    folder, name = os.path.split(ref_path)
    if not name.startswith("ref_"):
        raise ValueError("a reference file is named ref_<task>.<ext>")
    return os.path.join(folder, "empty_" + name[len("ref_"):])


def has_markers(ref_text: str) -> bool:
    return any(_OPEN.match(l) for l in ref_text.splitlines())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("reference")
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--drop-line-containing", action="append", default=[])
    args = ap.parse_args(argv)
    with open(args.reference) as f:
        ref_text = f.read()
    if not has_markers(ref_text):
        # Without markers the "skeleton" would be the whole solution: never write that.
        print(f"no solution markers in {args.reference}: its skeleton is kept by hand", file=sys.stderr)
        return 2
    text = skeleton_text(ref_text, tuple(args.drop_line_containing))
    path = skeleton_path(args.reference)
    if args.check:
        with open(path) as f:
            same = f.read() == text
        print(("up to date: " if same else "DIFFERS: ") + path)
        return 0 if same else 1
    with open(path, "w") as f:
        f.write(text)
    print(path)
    return 0


if __name__ == "__main__":
    sys.exit(main())
