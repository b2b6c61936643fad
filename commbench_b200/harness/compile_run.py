"""Build and run one candidate program of a task, under a hard time limit, and read its result.

A *task* is a folder with a skeleton (``empty_<name>.<ext>``), a reference implementation
(``ref_<name>.<ext>``) and ``task.json`` (how to launch: plain python, ``torchrun`` with W ranks,
or an ``nvcc``-built binary).  A *candidate* is any source file that fills the skeleton.  A
candidate prints ONE JSON object on stdout (``{"Correctness": "PASS", ..., "metrics": [...]}``)
and may print a ``METRICS_JSON: {...}`` line.

Counterpart of the reference's ``run_eval/compile_run.py``: scrubbed build environment
(:92-153), process-group kill on time-out and on normal exit so leaked rank workers cannot keep
a GPU busy (:156-199), ``CompileRunResult`` (:208-271), skeleton / reference look-up over the
known extensions (:336-409), ``METRICS_JSON`` parsing (:412-443), pass/fail analysis
(:519-555), error summary for the next prompt (:558-599), ``compile_and_run`` (:602-751) and
the reference-vs-candidate comparison (:754-819).  CUDA candidates are compiled for sm_100a only,
with this package's ``csrc`` on the include path, so they can use its bounded-wait primitives.
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
import time
from dataclasses import asdict, dataclass, field

from ..runtime.launcher import run_in_new_session
from . import verdict as V

SOURCE_EXTS = (".py", ".cu", ".cpp", ".cc", ".cxx")
PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REPO_ROOT = os.path.dirname(PKG_ROOT)
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++20", "-O3", "-lineinfo",
              "--expt-relaxed-constexpr", "-Xptxas=-v,--warn-on-spills"]
NVCC_DEBUG_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++20", "-O0", "-g", "-G",
                    "--expt-relaxed-constexpr"]


@dataclass
class CompileRunResult:
    source: str
    compile_success: bool = False
    compile_returncode: int | None = None
    compile_output: str = ""
    run_success: bool = False
    run_returncode: int | None = None
    run_stdout: str = ""
    run_stderr: str = ""
    timed_out: bool = False
    wall_s: float = 0.0
    result_json: dict | None = None
    metrics: dict = field(default_factory=dict)
    command: list[str] = field(default_factory=list)
    ptxas: list = field(default_factory=list)      # per kernel: registers, spills, static smem

    def to_dict(self) -> dict:
        return asdict(self)

    @property
    def output(self) -> str:
        return "\n".join(x for x in (self.compile_output, self.run_stdout, self.run_stderr) if x)


def scrubbed_env(extra: dict | None = None) -> dict:
    """Environment for builds and runs: no conda / virtualenv compiler overrides, CUDA_HOME pinned
    to the toolkit whose nvcc is used, the package importable, rendezvous on 127.0.0.1."""
    env = dict(os.environ)
    for k in list(env):
        if k.startswith("CONDA_") or k in ("CC", "CXX", "CFLAGS", "CXXFLAGS", "LDFLAGS", "NVCC_PREPEND_FLAGS",
                                           "NVCC_APPEND_FLAGS", "TORCH_CUDA_ARCH_LIST"):
            env.pop(k)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if os.path.exists(nvcc):
        env["CUDA_HOME"] = os.path.dirname(os.path.dirname(os.path.realpath(nvcc)))
        env["PATH"] = os.path.dirname(nvcc) + os.pathsep + env.get("PATH", "")
    env["PYTHONPATH"] = REPO_ROOT + os.pathsep + env.get("PYTHONPATH", "")
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    if extra:
        env.update({k: str(v) for k, v in extra.items()})
    return env


def load_task(folder: str) -> dict:
    """``task.json`` with defaults filled in."""
    spec = {"name": os.path.basename(os.path.normpath(folder)), "launcher": "python", "world": 1,
            "timeout_s": 180, "op": None, "args": [], "needs_gpu": False, "env": {}}
    p = os.path.join(folder, "task.json")
    if os.path.exists(p):
        with open(p) as f:
            spec.update(json.load(f))
    return spec


PLATFORM_SUBDIRS = ("nv", "ib", "roce", "efa")


def platform_subdir_order(platform: str | None = None) -> list[str]:
    """Where a task keeps its files: the folder itself, or a per-platform sub-folder
    (``nv`` for the GPU vendor, then the fabric this machine has: ``ib`` / ``roce`` / ``efa``; a
    machine without a NIC still finds the ``ib`` variants, which run on the loopback transport).
    The reference resolves ``amd_nv -> amd / nv -> ib, roce / efa``
    (run_eval/compile_run.py:274-333); there is one GPU vendor here."""
    order = ["", "nv"]
    p = (platform or "").upper()
    for net in ("ib", "roce", "efa"):
        if net.upper() in p:
            order.append(net)
    for net in ("ib", "roce", "efa"):
        if net not in order:
            order.append(net)
    return order


def _find(folder: str, prefix: str, platform: str | None = None) -> str | None:
    for sub in platform_subdir_order(platform):
        d = os.path.join(folder, sub) if sub else folder
        if not os.path.isdir(d):
            continue
        hits = sorted(f for f in os.listdir(d) if f.startswith(prefix) and f.endswith(SOURCE_EXTS))
        if hits:
            return os.path.join(d, hits[0])
    return None


def find_empty_file(folder: str, platform: str | None = None) -> str | None:
    return _find(folder, "empty_", platform)


def find_ref_file(folder: str, platform: str | None = None) -> str | None:
    return _find(folder, "ref_", platform)


def first_json_object(text: str) -> dict | None:
    """The first balanced ``{...}`` of ``text`` that parses as JSON (programs may log around it)."""
    start = text.find("{")
    while start != -1:
        depth, in_str, esc = 0, False, False
        for i in range(start, len(text)):
            c = text[i]
            if in_str:
                if esc:
                    esc = False
                elif c == "\\":
                    esc = True
                elif c == '"':
                    in_str = False
                continue
            if c == '"':
                in_str = True
            elif c == "{":
                depth += 1
            elif c == "}":
                depth -= 1
                if depth == 0:
                    try:
                        obj = json.loads(text[start:i + 1])
                        if isinstance(obj, dict):
                            return obj
                    except json.JSONDecodeError:
                        pass
                    break
        start = text.find("{", start + 1)
    return None


def extract_metrics(output: str) -> dict:
    for line in (output or "").splitlines():
        line = line.strip()
        if line.startswith("METRICS_JSON:"):
            try:
                m = json.loads(line[len("METRICS_JSON:"):].strip())
                if isinstance(m, dict):
                    return m
            except json.JSONDecodeError:
                continue
    return {}


def build_command(spec: dict, source: str, binary: str | None) -> list[str]:
    args = [str(a) for a in spec.get("args", [])]
    launcher = spec["launcher"]
    if launcher == "python":
        return [sys.executable, source] + args
    if launcher == "torchrun":
        from ..runtime.launcher import free_port

        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                f"--nproc-per-node={int(spec['world'])}", "--master-addr", "127.0.0.1",
                "--master-port", str(free_port()), source] + args
    if launcher == "nvcc":
        return [binary] + args
    raise ValueError(f"unknown launcher {launcher!r}")


def ptxas_report(log: str) -> list[dict]:
    """Per kernel: registers, spill bytes and static shared memory out of a ``ptxas -v`` log."""
    import re

    out, cur = [], None
    for line in log.splitlines():
        m = re.search(r"Compiling entry function '([^']+)'", line)
        if m:
            cur = {"kernel": m.group(1), "registers": None, "spill_stores": 0, "spill_loads": 0,
                   "smem_bytes": 0}
            out.append(cur)
            continue
        if cur is None:
            continue
        m = re.search(r"(\d+) bytes spill stores, (\d+) bytes spill loads", line)
        if m:
            cur["spill_stores"], cur["spill_loads"] = int(m.group(1)), int(m.group(2))
        m = re.search(r"Used (\d+) registers", line)
        if m:
            cur["registers"] = int(m.group(1))
            s = re.search(r"(\d+) bytes smem", line)
            cur["smem_bytes"] = int(s.group(1)) if s else 0
    return out


def _source_digest(source: str, flags: list[str]) -> str:
    import hashlib

    h = hashlib.sha256(" ".join(flags).encode())
    with open(source, "rb") as f:
        h.update(f.read())
    return h.hexdigest()


def compile_source(source: str, out_dir: str, timeout_s: float = 300.0,
                   debug: bool = False) -> tuple[bool, int | None, str, str | None]:
    """(ok, returncode, log, binary).  Python sources are byte-compiled as the syntax check.
    CUDA / C++ sources are built with nvcc for sm_100a; the log carries the ``ptxas -v`` report
    (registers, spills; ``debug`` builds ``-O0 -g -G`` instead).  A binary whose source text and
    flags have not changed since it was built in ``out_dir`` is reused (the log is kept beside
    it), like the reference's mtime binary cache
    (datasets/example060_thunderkitten_all_reduce_hard/nv/build_and_run.py:227-242)."""
    ext = os.path.splitext(source)[1]
    if ext == ".py":
        r = run_in_new_session([sys.executable, "-m", "py_compile", source], timeout=60,
                               env=scrubbed_env())
        return r.returncode == 0, r.returncode, (r.stdout + r.stderr), None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        return False, None, "nvcc not found", None
    os.makedirs(out_dir, exist_ok=True)
    binary = os.path.join(out_dir, os.path.splitext(os.path.basename(source))[0])
    flags = NVCC_DEBUG_FLAGS if debug else NVCC_FLAGS
    digest, stamp = _source_digest(source, flags), binary + ".build.json"
    if os.path.exists(binary) and os.path.exists(stamp):
        try:
            with open(stamp) as f:
                old = json.load(f)
            if old.get("digest") == digest:
                return True, 0, old.get("log", "") + "\n[build cache hit]", binary
        except (OSError, json.JSONDecodeError):
            pass
    cmd = [nvcc] + flags + ["-I", os.path.join(PKG_ROOT, "csrc"), "-x", "cu", source, "-o", binary,
                            "-lcuda"]
    r = run_in_new_session(cmd, timeout=timeout_s, env=scrubbed_env())
    ok = r.returncode == 0 and os.path.exists(binary)
    log = r.stdout + r.stderr
    if ok:
        with open(stamp, "w") as f:
            json.dump({"digest": digest, "log": log}, f)
    return ok, r.returncode, log, binary if ok else None


def compile_and_run(folder: str, source: str, timeout_s: float | None = None,
                    build_only: bool = False, work_dir: str | None = None) -> CompileRunResult:
    # The program runs with the task folder as its working directory: relative paths given by the
    # caller must not be re-interpreted there.
    folder, source = os.path.abspath(folder), os.path.abspath(source)
    spec = load_task(folder)
    res = CompileRunResult(source=source)
    work_dir = os.path.abspath(work_dir) if work_dir else os.path.join(folder, "build")
    t0 = time.time()
    ok, rc, log, binary = compile_source(source, work_dir, debug=bool(spec.get("debug")))
    res.compile_success, res.compile_returncode, res.compile_output = ok, rc, log
    res.ptxas = ptxas_report(log)
    if not ok or build_only:
        res.wall_s = time.time() - t0
        return res
    cmd = build_command(spec, source, binary)
    res.command = cmd
    r = run_in_new_session(cmd, timeout=float(timeout_s or spec["timeout_s"]),
                           env=scrubbed_env(spec.get("env")), cwd=folder)
    res.run_returncode, res.run_stdout, res.run_stderr = r.returncode, r.stdout, r.stderr
    res.timed_out = r.timed_out
    res.run_success = (r.returncode == 0) and not r.timed_out
    res.result_json = first_json_object(r.stdout)
    res.metrics = extract_metrics(r.stdout + "\n" + r.stderr)
    res.wall_s = time.time() - t0
    return res


def analyze_result(res: CompileRunResult) -> tuple[bool, str]:
    if not res.compile_success:
        return False, f"build failed (rc={res.compile_returncode})"
    if res.timed_out:
        return False, "run timed out"
    if not res.run_success:
        return False, f"run failed (rc={res.run_returncode})"
    j = res.result_json or {}
    verdict_field = str(j.get("Correctness", j.get("correctness", ""))).upper()
    if verdict_field == "FAIL" or "FAIL" in res.run_stdout or "FAIL" in res.run_stderr:
        return False, "program reported FAIL"
    if verdict_field == "PASS" or "PASS" in res.run_stdout:
        return True, "program reported PASS"
    return True, "ran to completion (no explicit verdict)"


def get_error_details(res: CompileRunResult, limit: int = 1500) -> str:
    """The part of the logs worth showing to whoever fixes the candidate (tail-biased)."""
    if not res.compile_success:
        text = res.compile_output
        head = "Build error:\n"
    elif res.timed_out:
        text = (res.run_stdout + "\n" + res.run_stderr)
        head = "Run exceeded its time limit; last output:\n"
    else:
        text = (res.run_stderr or "") + ("\n" + res.run_stdout if res.run_stdout else "")
        head = f"Run failed (rc={res.run_returncode}):\n"
    text = text.strip()
    if len(text) > limit:
        text = "...\n" + text[-limit:]
    return head + text


def metrics_average(result_json: dict | None) -> dict:
    """``{data_size_avg, latency_avg, throughput_avg}`` over the ``metrics`` list of a result."""
    rows = (result_json or {}).get("metrics") or []
    out = {}
    for key, name in (("data_size", "data_size_avg"), ("latency_avg", "latency_avg"),
                      ("throughput_avg", "throughput_avg")):
        vals = [float(r[key]) for r in rows if isinstance(r, dict) and key in r]
        if vals:
            out[name] = sum(vals) / len(vals)
    return out


def compare_save_results(folder: str, ref_source: str, gen_source: str, results_dir: str,
                         timeout_s: float | None = None) -> dict:
    """Runs reference then candidate back to back, writes ``summary.json`` in ``results_dir`` with
    both results, the per-metric comparison and the unified verdict."""
    spec = load_task(folder)
    os.makedirs(results_dir, exist_ok=True)
    ref = compile_and_run(folder, ref_source, timeout_s, work_dir=os.path.join(results_dir, "build_ref"))
    gen = compile_and_run(folder, gen_source, timeout_s, work_dir=os.path.join(results_dir, "build_gen"))
    ref_m = {**metrics_average(ref.result_json), **ref.metrics}
    gen_m = {**metrics_average(gen.result_json), **gen.metrics}
    # The task names the metric its programs print; otherwise the op registry decides.
    entry = None
    if spec.get("primary_metric"):
        entry = {"primary": spec["primary_metric"], "direction": spec.get("direction", "lower")}
    elif spec.get("op"):
        from . import registry

        entry = registry.entry(spec["op"])
    v = V.compute_verdict(entry if entry is not None else "info_only", ref_m, gen_m)
    gen_ok, gen_why = analyze_result(gen)
    units = {k: (gen.result_json or ref.result_json or {}).get(k)
             for k in ("data_size_unit", "latency_unit", "throughput_unit")}

    def side(r: CompileRunResult) -> dict:
        regs = [p["registers"] for p in r.ptxas if p.get("registers") is not None]
        return {"compile_success": r.compile_success, "run_success": r.run_success,
                "timed_out": r.timed_out, "wall_s": round(r.wall_s, 3),
                "max_registers": max(regs) if regs else None,
                "spill_bytes": sum(p["spill_stores"] + p["spill_loads"] for p in r.ptxas)}

    summary = {
        "task": spec["name"],
        "ref_source": os.path.basename(ref_source),
        "generated_source": os.path.basename(gen_source),
        **units,
        "build_and_run": {"reference": side(ref), "generated": side(gen)},
        "verdict_scheme": {"better_pct": V.BETTER_PCT, "on_par_lower_pct": V.ON_PAR_LOWER_PCT,
                           "degraded_lower_pct": V.DEGRADED_LOWER_PCT},
        "correctness": {"reference": analyze_result(ref)[0], "generated": gen_ok, "reason": gen_why},
        "metrics_comparison": {k: {"reference": ref_m.get(k), "generated": gen_m.get(k)}
                               for k in sorted(set(ref_m) | set(gen_m))},
        "performance": v.verdict,
        "performance_detail": v.detail,
    }
    with open(os.path.join(results_dir, "summary.json"), "w") as f:
        json.dump(summary, f, indent=1)
    for tag, r in (("ref", ref), ("gen", gen)):
        with open(os.path.join(results_dir, f"{tag}_output.txt"), "w") as f:
            f.write(r.output)
    return summary
