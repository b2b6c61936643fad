"""Per-rank process launch with session-group clean-up.

``run_ranks`` starts ``torch.distributed.run`` (one process per GPU, rendezvous on
127.0.0.1) in a NEW POSIX session and kills the whole session group on time-out
*and* after a normal exit, so a leaked rank worker can never keep spinning on a
GPU.  Same containment as the reference's ``_run_in_new_session``
(run_eval/compile_run.py:156-199) and its fork-per-GPU mains with
``PR_SET_PDEATHSIG`` (datasets/example060_thunderkitten_all_reduce_hard/nv/
empty_thunderkitten_all_reduce.cu:524-580).
"""
from __future__ import annotations

import os
import signal
import socket
import subprocess
import sys
import time
from dataclasses import dataclass


@dataclass
class RunResult:
    returncode: int
    stdout: str
    stderr: str
    timed_out: bool
    seconds: float


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _kill_group(pgid: int):
    for sig in (signal.SIGTERM, signal.SIGKILL):
        try:
            os.killpg(pgid, sig)
        except ProcessLookupError:
            return
        except PermissionError:
            return
        time.sleep(0.5)


def die_with_parent(sig: int = signal.SIGKILL) -> bool:
    """Asks the kernel to send ``sig`` to THIS process when its parent dies
    (``prctl(PR_SET_PDEATHSIG)``): a rank worker then cannot outlive a launcher that was killed
    before it could clean up.  Returns False where the call is not available."""
    prctl = _prctl()
    return prctl is not None and prctl(1, int(sig), 0, 0, 0) == 0     # 1 = PR_SET_PDEATHSIG


_PRCTL = None


def _prctl():
    """libc's prctl, looked up once in the parent: the child of a fork must not import anything
    (another thread may have held the import lock at the time of the fork)."""
    global _PRCTL
    if _PRCTL is None:
        try:
            import ctypes

            _PRCTL = ctypes.CDLL(None, use_errno=True).prctl
        except (OSError, AttributeError):
            _PRCTL = False
    return _PRCTL or None


def run_in_new_session(cmd: list[str], timeout: float, env: dict | None = None,
                       cwd: str | None = None, pdeathsig: bool = True) -> RunResult:
    """Runs ``cmd`` in a new session; the whole session group is killed on time-out and after a
    normal exit.  With ``pdeathsig`` the child is also killed when this process dies first."""
    t0 = time.time()
    # Python code between fork and exec is kept out of parents that hold a CUDA context (many
    # driver threads): there the session-group kill below is the containment.
    torch_mod = sys.modules.get("torch")
    cuda_live = bool(torch_mod is not None and torch_mod.cuda.is_initialized())
    use_pd = pdeathsig and not cuda_live and _prctl() is not None
    p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                         start_new_session=True, env=env, cwd=cwd,
                         preexec_fn=die_with_parent if use_pd else None)
    timed_out = False
    try:
        out, err = p.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        timed_out = True
        _kill_group(p.pid)
        out, err = p.communicate()
    finally:
        # Also after a normal exit: nothing of that session may survive.
        _kill_group(p.pid)
    return RunResult(p.returncode if p.returncode is not None else -9, out, err, timed_out,
                     time.time() - t0)


def run_ranks(script: str, nproc: int, args: list[str] | None = None, timeout: float = 600.0,
              env_extra: dict | None = None, cwd: str | None = None) -> RunResult:
    """Runs ``script`` as ``nproc`` ranks of one node."""
    env = dict(os.environ)
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    if env_extra:
        env.update({k: str(v) for k, v in env_extra.items()})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), script, *(args or [])]
    return run_in_new_session(cmd, timeout, env=env, cwd=cwd)
