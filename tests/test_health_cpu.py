"""Failure detection and recovery, with failures made on the host only."""
import json
import os
import subprocess
import sys
import time

import pytest

from commbench_b200.runtime import health as H

HERE = os.path.dirname(os.path.abspath(__file__))


def _spawn(case, world, scratch):
    return [subprocess.Popen([sys.executable, os.path.join(HERE, "health_cases.py"), case, str(r),
                              str(world), str(scratch)], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                             text=True) for r in range(world)]


def _join(procs, timeout):
    outs = []
    deadline = time.time() + timeout
    for p in procs:
        try:
            o, e = p.communicate(timeout=max(1.0, deadline - time.time()))
        except subprocess.TimeoutExpired:
            p.kill()                         # exactly this child, by handle
            o, e = p.communicate()
            e += "\n[killed: timed out]"
        outs.append((p.returncode, o, e))
    return outs


def _results(scratch, ranks):
    out = {}
    for r in ranks:
        p = os.path.join(scratch, f"result_rank{r}.json")
        if os.path.exists(p):
            out[r] = json.load(open(p))
    return out


def test_board_and_watchdog_in_one_process(tmp_path):
    name = f"cb_health_unit_{os.getpid()}"
    a = H.HeartbeatBoard(name, 0, 2, interval_s=0.01)
    b = H.HeartbeatBoard(name, 1, 2, interval_s=0.01, create=False)
    a.wait_all_present(5)
    wd = H.Watchdog(a, timeout_s=0.2)
    time.sleep(0.05)
    assert wd.dead_ranks() == []
    wd.check()
    b._stop.set()                            # rank 1 stops beating without a word
    assert wd.wait_for_failure(2.0) == [1]
    with pytest.raises(H.RankFailure) as ei:
        wd.check()
    assert ei.value.dead == [1]
    b.leave(failed=True, err=7)
    assert a.read(1)[2] == H.FAILED and a.read(1)[3] == 7
    assert H.survivors_of(4, [1, 3]) == [0, 2]
    assert not H._pid_alive(0) and H._pid_alive(os.getpid())
    b.close()
    a.close(unlink=True)


@pytest.mark.timeout(240)
@pytest.mark.parametrize("case", ["cpu_elastic", "cpu_elastic_silent"])
def test_rank_leaves_survivors_rerendezvous(tmp_path, case):
    scratch = tmp_path / "s"
    scratch.mkdir()
    outs = _join(_spawn(case, 3, scratch), 180)
    res = _results(scratch, [0, 1, 2])
    assert set(res) >= {0, 1}, outs
    for r in (0, 1):
        assert res[r]["step1"] == 6.0                      # 1 + 2 + 3 with all three ranks
        assert res[r]["dead"] == [2] and res[r]["raised"]
        assert res[r]["new_world"] == 2 and res[r]["new_rank"] == r
        assert res[r]["step2"] == 3.0                      # 1 + 2 with the survivors
    assert all(rc == 0 for rc, _, _ in outs), outs


@pytest.mark.timeout(240)
@pytest.mark.parametrize("case", ["cpu_runner", "cpu_runner_silent"])
def test_elastic_runner_shrinks_twice_and_finishes(tmp_path, case):
    """Four ranks, eight steps; rank 3 goes after step 2 and rank 1 after step 5.  The membership
    barrier keeps everybody out of a collective with a rank that is not coming."""
    scratch = tmp_path / "s"
    scratch.mkdir()
    outs = _join(_spawn(case, 4, scratch), 200)
    res = _results(scratch, [0, 1, 2, 3])
    assert set(res) == {0, 1, 2, 3}, outs
    assert res[3]["sums"] == [4, 4, 4] and res[3]["left_after"] == 2
    assert res[1]["sums"] == [4, 4, 4, 3, 3, 3] and res[1]["left_after"] == 5
    for r in (0, 2):
        assert res[r]["sums"] == [4, 4, 4, 3, 3, 3, 2, 2], (r, res[r], outs)
        assert [h["dead"] for h in res[r]["history"]] == [[3], [1]]
        assert [h["step"] for h in res[r]["history"]] == [3, 6]
        assert res[r]["members"] == [0, 2] and res[r]["final"] == [0 if r == 0 else 1, 2]
        # (generation, new rank, new world) seen by the caller's hook: old rank 2 becomes 1 at the end
        assert [tuple(x) for x in res[r]["reconfigured"]] == [(1, r, 3), (2, 0 if r == 0 else 1, 2)]
    assert all(rc == 0 for rc, _, _ in outs), outs


def test_membership_barrier_reports_a_rank_that_is_alive_but_stuck(tmp_path):
    name = f"cb_runner_unit_{os.getpid()}"
    a = H.HeartbeatBoard(name, 0, 2, interval_s=0.01)
    b = H.HeartbeatBoard(name, 1, 2, interval_s=0.01, create=False)
    a.wait_all_present(5)
    assert a.step_of(1) == -1
    b.announce_step(4)
    assert a.step_of(1) == 4
    r = H.ElasticRunner(name, 0, 2, str(tmp_path / "store"))
    r.board, r.watchdog = a, H.Watchdog(a, timeout_s=0.3)
    assert r.membership_barrier(4, timeout_s=1.0) == []          # the peer is already there
    with pytest.raises(H.RankFailure, match="never reached step 5"):
        r.membership_barrier(5, timeout_s=0.2)                   # beating, but not coming
    b.leave()
    assert r.membership_barrier(5, timeout_s=1.0) == [1]         # gone: reported, not waited for
    b.close()
    a.close(unlink=True)


@pytest.mark.gpu
@pytest.mark.timeout(300)
def test_gpu_rank_leaves_between_steps_peer_raises_before_launch(tmp_path, native_lib):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    scratch = tmp_path / "g"
    scratch.mkdir()
    outs = _join(_spawn("gpu_leave", 2, scratch), 240)
    res = _results(scratch, [0, 1])
    assert set(res) == {0, 1}, outs
    assert res[0]["step1"] == 3.0 and res[1]["step1"] == 3.0
    assert res[0]["dead"] == [1] and res[0]["launched"] is False and res[0]["status"] == 0
    assert res[1]["left"] is True
