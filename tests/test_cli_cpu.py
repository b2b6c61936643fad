"""``python -m commbench_b200 <command>``: the front door to the command-line tools."""
import importlib
import os
import subprocess
import sys

import commbench_b200.__main__ as M

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_command_resolves_to_a_module_with_an_entry():
    for cmd, modname in M.COMMANDS.items():
        mod = importlib.import_module(modname)
        assert hasattr(mod, "main") or cmd in ("examples", "build"), cmd
    assert M.main([]) == 0 and M.main(["help"]) == 0 and M.main(["no-such-command"]) == 2


def test_subcommands_run_in_a_fresh_interpreter(tmp_path):
    def run(*args):
        return subprocess.run([sys.executable, "-m", "commbench_b200", *args], cwd=ROOT, text=True,
                              capture_output=True, timeout=120)

    r = run("examples")
    rows = [l.split("|")[1].strip() for l in r.stdout.splitlines() if l.startswith("| example")]
    assert r.returncode == 0 and len(set(rows)) == 101          # one example may serve two ops
    r = run("platform", "--quiet")
    assert r.returncode == 0 and r.stdout.strip() in ("CPU", "NV", "NV_IB", "NV_ROCE", "NV_EFA")
    r = run("eval", "--list-tasks")
    assert r.returncode == 0 and "gloo_allreduce" in r.stdout.split()
    tasks = os.path.join("commbench_b200", "harness", "tasks")
    r = run("skeleton", os.path.join(tasks, "rdma_memory_pool", "ref_rdma_memory_pool.py"), "--check")
    assert r.returncode == 0 and r.stdout.startswith("up to date")
    r = run("skeleton", os.path.join(tasks, "rdma_atomics", "ref_rdma_atomics.py"))   # no markers
    assert r.returncode == 2 and "kept by hand" in r.stderr                          # nothing is written
    r = run("leaderboard", "--tasks-dir", str(tmp_path))
    assert r.returncode == 0 and r.stdout.startswith("| model |")
    r = run("build")
    assert r.returncode == 0 and r.stdout.strip().endswith("libcommbench_b200.so")
