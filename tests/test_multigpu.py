"""Real multi-GPU checks: rank processes over NCCL + our symmetric-memory kernels."""
import json
import os

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _nproc():
    n = torch.cuda.device_count()
    return 8 if n >= 8 else (4 if n >= 4 else 2)


def test_multi_rank_collectives_and_fused_ops(native_lib):
    from commbench_b200.runtime.launcher import run_ranks

    res = run_ranks(os.path.join(HERE, "mp_cases.py"), _nproc(), timeout=900)
    lines = [json.loads(l) for l in res.stdout.splitlines() if l.startswith("{")]
    failed = [l for l in lines if l.get("ok") is False]
    assert not res.timed_out, res.stderr[-2000:]
    assert not failed, failed
    assert res.returncode == 0, res.stderr[-2000:]
    assert any(l.get("summary") == "PASS" for l in lines)
