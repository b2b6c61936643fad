"""CPU-only tests of the host plumbing: broker (fd exchange, barrier, all-gather over shared
memory), shared-memory object broadcast, gloo all-reduce correctness, launcher clean-up."""
import ctypes as C
import multiprocessing as mp
import os
import sys
import uuid

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))


def _broker_worker(name, rank, world, q):
    from commbench_b200 import _native as N

    lib = N.load()
    b = C.c_void_p(0)
    assert lib.cb_broker_create(name.encode(), rank, world, 120000, C.byref(b)) == 0, N.last_error()
    # each rank contributes a memfd holding its rank number
    fd = os.memfd_create(f"r{rank}")
    os.write(fd, bytes([rank + 65]) * 8)
    fds = (C.c_int * 8)()
    for rnd in range(3):    # several rounds: out-of-order arrivals are stashed per round
        assert lib.cb_broker_exchange_fds(b, fd, fds, 120000) == 0, N.last_error()
        got = []
        for r in range(world):
            # pread: the descriptors share one file offset across all the processes
            got.append(os.pread(fds[r], 8, 0))
            os.close(fds[r])
        assert got == [bytes([r + 65]) * 8 for r in range(world)]
    assert lib.cb_broker_barrier(b, 120000) == 0
    mine = (C.c_ubyte * 16)(*([rank] * 16))
    allb = (C.c_ubyte * (16 * world))()
    assert lib.cb_broker_allgather(b, mine, 16, allb, 120000) == 0
    assert list(allb) == [r for r in range(world) for _ in range(16)]
    out = C.c_int(-1)
    assert lib.cb_broker_broadcast_fd(b, 1, fd, C.byref(out), 120000) == 0
    assert os.pread(out.value, 8, 0) == bytes([1 + 65]) * 8
    os.close(out.value)
    lib.cb_broker_destroy(b)
    q.put((rank, "ok"))


@pytest.mark.parametrize("world", [2, 4])
def test_broker_fd_exchange_barrier_allgather(native_lib, world):
    name = "cbt-" + uuid.uuid4().hex[:10]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_broker_worker, args=(name, r, world, q)) for r in range(world)]
    for p in ps:
        p.start()
    for p in ps:
        p.join(300)
        assert p.exitcode == 0
    assert sorted(q.get(timeout=5)[0] for _ in range(world)) == list(range(world))


def test_broker_barrier_times_out_when_a_rank_never_joins(native_lib):
    """Failure made on the host: rank 1 never arrives; rank 0 must get an error, not hang."""
    from commbench_b200 import _native as N

    lib = N.load()
    b = C.c_void_p(0)
    name = "cbt-" + uuid.uuid4().hex[:10]
    assert lib.cb_broker_create(name.encode(), 0, 2, 5000, C.byref(b)) == 0
    assert lib.cb_broker_barrier(b, 200) == -2
    assert "timed out" in N.last_error()
    lib.cb_broker_destroy(b)


def _shm_reader(name, idx, n_msgs, q):
    from commbench_b200.ops.util import ShmBroadcast

    r = ShmBroadcast(name, n_readers=2, reader_index=idx)
    out = [r.dequeue(timeout_ms=120000) for _ in range(n_msgs)]
    r.close()
    q.put((idx, out))


def test_shm_broadcast_objects_small_and_multi_slot(native_lib):
    from commbench_b200.ops.util import ShmBroadcast

    name = "cbq-" + uuid.uuid4().hex[:10]
    w = ShmBroadcast(name, n_readers=2, nslots=4, slot_bytes=4096)
    msgs = [{"step": i, "blob": bytes([i % 251]) * (100 + 3000 * i)} for i in range(12)]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_shm_reader, args=(name, i, len(msgs), q)) for i in range(2)]
    for p in ps:
        p.start()
    for m in msgs:
        w.broadcast_object(m, timeout_ms=120000)
    res = dict(q.get(timeout=300) for _ in range(2))
    for p in ps:
        p.join(30)
    w.close()
    assert res[0] == msgs and res[1] == msgs


def test_shm_dequeue_times_out(native_lib):
    from commbench_b200.ops.util import ShmBroadcast

    name = "cbq-" + uuid.uuid4().hex[:10]
    w = ShmBroadcast(name, n_readers=1)
    r = ShmBroadcast(name, n_readers=1, reader_index=0)
    with pytest.raises(TimeoutError):
        r.dequeue(timeout_ms=100)
    r.close()
    w.close()


def _gloo_allreduce(rank, world, port, q):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(rank)
    x = torch.randn(1_048_576, generator=g, dtype=torch.float32)
    ref = torch.zeros(1_048_576, dtype=torch.float64)
    for r in range(world):
        ref += torch.randn(1_048_576, generator=torch.Generator().manual_seed(r),
                           dtype=torch.float32).double()
    dist.all_reduce(x)
    ok = torch.allclose(x.double(), ref, rtol=1e-5, atol=1e-5)
    dist.destroy_process_group()
    q.put((rank, bool(ok)))


def test_gloo_sum_all_reduce_matches_fp64(native_lib):
    """world_size=2 on CPU: fp32 N(0,1) tensors of 1,048,576 elements seeded by rank, checked
    against an fp64 sum with rtol 1e-5."""
    from commbench_b200.runtime.launcher import free_port

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    ps = [ctx.Process(target=_gloo_allreduce, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in ps:
        p.join(30)
    assert res == {0: True, 1: True}


def test_launcher_kills_session_on_timeout(tmp_path):
    from commbench_b200.runtime.launcher import run_in_new_session

    script = tmp_path / "sleeper.py"
    script.write_text("import time, subprocess, sys\n"
                      "subprocess.Popen([sys.executable, '-c', 'import time; time.sleep(60)'])\n"
                      "time.sleep(60)\n")
    r = run_in_new_session([sys.executable, str(script)], timeout=1.0)
    assert r.timed_out
    assert r.seconds < 10


def test_rank_worker_dies_with_a_launcher_that_was_killed(tmp_path):
    """A launcher killed with SIGKILL cannot clean up; its worker asked the kernel to be killed
    when the parent dies, so nothing is left behind."""
    import signal
    import subprocess
    import time

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pidfile = tmp_path / "worker.pid"
    worker = tmp_path / "worker.py"
    worker.write_text(f"import os, time\nopen({str(pidfile)!r}, 'w').write(str(os.getpid()))\ntime.sleep(120)\n")
    launcher = tmp_path / "launcher.py"
    launcher.write_text(
        f"import sys\nsys.path.insert(0, {repo!r})\n"
        "from commbench_b200.runtime.launcher import run_in_new_session\n"
        f"run_in_new_session([sys.executable, {str(worker)!r}], timeout=100)\n")
    p = subprocess.Popen([sys.executable, str(launcher)])
    deadline = time.time() + 30
    while not (pidfile.exists() and pidfile.read_text().strip()) and time.time() < deadline:
        time.sleep(0.05)
    wpid = int(pidfile.read_text())
    os.kill(p.pid, signal.SIGKILL)                     # exactly the launcher we started
    p.wait(10)

    def alive(pid):
        try:
            with open(f"/proc/{pid}/stat") as f:
                return f.read().rsplit(")", 1)[1].split()[0] != "Z"
        except OSError:
            return False

    deadline = time.time() + 10
    while alive(wpid) and time.time() < deadline:
        time.sleep(0.05)
    gone = not alive(wpid)
    if not gone:
        os.kill(wpid, signal.SIGKILL)                  # do not leave it behind if the check fails
    assert gone


def test_gate_up_interleave_puts_both_halves_of_an_output_block_in_one_tile():
    """Row order the gated up-projection epilogue expects: per block of 128 outputs the gate
    rows, then the up rows of the same outputs."""
    from commbench_b200.ops.moe import interleave_gate_up

    E, I, H = 3, 256, 16
    w1 = torch.arange(E * 2 * I * H, dtype=torch.float32).reshape(E, 2 * I, H)
    out = interleave_gate_up(w1)
    assert out.shape == w1.shape and out.is_contiguous()
    for e in range(E):
        for j in range(I // 128):
            tile = out[e, j * 256:(j + 1) * 256]
            assert torch.equal(tile[:128], w1[e, j * 128:(j + 1) * 128])
            assert torch.equal(tile[128:], w1[e, I + j * 128:I + (j + 1) * 128])
    x = torch.randn(5, H)
    h = x @ w1[1].t()
    ref = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
    hg = (x @ out[1].t()).reshape(5, I // 128, 2, 128)
    assert torch.allclose((torch.nn.functional.silu(hg[:, :, 0]) * hg[:, :, 1]).reshape(5, I), ref)
    with pytest.raises(Exception):
        interleave_gate_up(torch.zeros(1, 2 * 96, 8))


def test_dispatch_rows_per_pair_and_per_token():
    """Rows a rank sends to each destination: one per selection, or one per (token, rank) couple;
    and the rule that picks the sender in the per-token form (the first selection of the token
    that lives on the rank) names exactly one selection of every couple."""
    from commbench_b200.ops.moe import dispatch_rows

    E, W, K = 16, 4, 4
    per = E // W
    idx = torch.tensor([[0, 1, 2, 3],          # all four on rank 0
                        [0, 4, 8, 12],         # one on each rank
                        [5, 6, 13, -1],        # two on rank 1, one on rank 3, one masked
                        [15, 14, 13, 12]])     # all four on rank 3
    assert dispatch_rows(idx, E, W, per_token=False) == [5, 3, 1, 6]
    assert dispatch_rows(idx, E, W, per_token=True) == [2, 2, 1, 3]
    owners = [0] * W
    for t in range(idx.shape[0]):
        for k in range(K):
            e = int(idx[t, k])
            if e < 0:
                continue
            d = e // per
            if not any(0 <= int(idx[t, kk]) and int(idx[t, kk]) // per == d for kk in range(k)):
                owners[d] += 1
    assert owners == dispatch_rows(idx, E, W, per_token=True)
    g = torch.Generator().manual_seed(0)
    big = torch.stack([torch.randperm(256, generator=g)[:8] for _ in range(512)])
    pair, tok = dispatch_rows(big, 256, 8, False), dispatch_rows(big, 256, 8, True)
    assert sum(pair) == 512 * 8 and all(t <= p for t, p in zip(tok, pair))
    assert 0.55 < sum(tok) / sum(pair) < 0.75        # 8 * (1 - (7/8)^8) / 8 = 0.66 expected
