"""FIFOs and probes on one GPU."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_d2h_fifo_all_triggers_arrive_once(native_lib):
    from commbench_b200.ops.util import D2HFifo

    f = D2HFifo(size=512)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    f.start_proxy()
    blocks, threads, per = 4, 256, 16
    f.push_test(blocks, threads, per, status=st)
    torch.cuda.synchronize()
    n = blocks * threads * per
    t0 = time.time()
    while f.popped() < n and time.time() - t0 < 10:
        time.sleep(0.001)
    popped, checksum, span_ns = f.stop_proxy()
    f.close()
    assert int(st.item()) == 0
    assert popped == n
    assert checksum == n * (n + 1) // 2      # every id 1..n exactly once


def test_d2h_fifo_push_times_out_without_consumer(native_lib):
    """Nothing pops: once the ring is full a push must give up and leave a status word."""
    from commbench_b200.ops.util import D2HFifo

    f = D2HFifo(size=8)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    f.push_test(1, 32, 1, timeout_s=0.05, status=st)
    torch.cuda.synchronize()
    assert (int(st.item()) >> 24) & 0xFF == 6     # CB_TIMEOUT_HOST_FLAG
    f.close()


def test_h2d_fifo_items_in_order(native_lib):
    from commbench_b200.ops.util import H2DFifo

    f = H2DFifo(size=16)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    n = 100
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        res = f.launch_consumer(n, timeout_s=5.0, status=st, stream=s)
    for i in range(n):
        f.push(1000 + i)
    s.synchronize()
    assert int(st.item()) == 0
    assert res[:, 0].tolist() == [1000 + i for i in range(n)]
    assert bool((res[1:, 1] >= res[:-1, 1]).all())
    f.close()


def test_probes(native_lib):
    from commbench_b200.ops import util

    attrs = util.device_attributes(0)
    assert attrs["sm_count"] > 0 and attrs["warp_size"] == 32
    src = torch.randint(0, 255, (64 << 20,), dtype=torch.uint8, device="cuda")
    dst = torch.empty_like(src)
    for w in (4, 8, 16):
        bw = util.copy_bandwidth(dst.data_ptr(), src.data_ptr(), src.numel(), width=w)
        assert bw > 100
    assert torch.equal(dst, src)
    ns = util.nanosleep_probe(10000)
    assert 5000 < ns["measured_ns"] < 200000
    mb = util.mbarrier_round_trip(threads=128, iters=1024)
    assert mb["cycles_per_iter"] > 0
    bw = util.tma_stream_bandwidth(src, tile_bytes=65536, stages=3, iters=64, blocks=148)
    assert bw > 100
    # D2H into pinned host memory: copy engine vs kernel stores into mapped memory
    host = torch.empty(16 << 20, dtype=torch.uint8).pin_memory()
    assert util.memcpy_bandwidth(host, src[:16 << 20]) > 1


def _ipc_consumer(handle, q):
    import torch

    from commbench_b200.ops.util import ipc_import

    w = ipc_import(handle)                       # maps the producer's allocation, no copy
    local = torch.empty_like(w)
    local.copy_(w)                               # "load the new weights"
    torch.cuda.synchronize()
    q.put((tuple(w.shape), float(local.double().sum().item()), int(w.data_ptr() != 0)))


@pytest.mark.timeout(300)
def test_ipc_weight_hand_off_between_two_processes(native_lib):
    """A trainer process exports a weight tensor by CUDA-IPC handle; an inference process on the
    same GPU maps it and copies it into its own weights (no host staging)."""
    import torch.multiprocessing as mp

    from commbench_b200.ops.util import ipc_export

    w = torch.arange(1 << 20, device="cuda", dtype=torch.float32).view(1024, 1024)
    expect = float(w.double().sum().item())
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_ipc_consumer, args=(ipc_export(w), q))
    p.start()
    shape, total, mapped = q.get(timeout=240)
    p.join(60)
    assert p.exitcode == 0 and shape == (1024, 1024) and mapped == 1
    assert total == expect


@pytest.mark.parametrize("shape", [(8,), (1000, 8), (4096, 8192), (3, 5)])
def test_abs_mean_one_pass_matches_torch(native_lib, shape):
    """The step metric: one launch, one pass; repeated calls re-arm the scratch words; shapes the
    kernel does not take (not a multiple of 8 elements) fall back to the PyTorch expression."""
    from commbench_b200.ops.util import abs_mean

    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(shape, device="cuda", generator=g).bfloat16()
    want = x.float().abs().mean().item()
    for _ in range(3):
        got = abs_mean(x)
        assert got.shape == (1,) and got.dtype == torch.float32
        assert abs(got.item() - want) <= 1e-4 * max(abs(want), 1e-6)
    out = torch.empty(1, device="cuda")
    assert abs_mean(x, out=out).data_ptr() == out.data_ptr()
    assert abs(out.item() - want) <= 1e-4 * max(abs(want), 1e-6)
