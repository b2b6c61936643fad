"""Fused TP QK-RMSNorm with virtual ranks, and the one-sided (put / get / signal / atomic /
tile) primitives, on one GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_emu_qknorm_matches_reference(native_lib, world):
    from commbench_b200.ops.fused import TPQKNorm, reference_qknorm
    from commbench_b200.runtime.context import EmuContext

    tokens, q_local, k_local = 37, 6144 // 8, 1024 // 8
    ctx = EmuContext(world)
    op = TPQKNorm(ctx, max_tokens=64, q_local=q_local, k_local=k_local, eps=1e-6)
    for call in range(3):        # three calls: both epochs and the slot clean-up
        g = torch.Generator(device="cuda").manual_seed(call)
        q = [torch.randn(tokens, q_local, device="cuda", generator=g).bfloat16() for _ in range(world)]
        k = [torch.randn(tokens, k_local, device="cuda", generator=g).bfloat16() for _ in range(world)]
        wq = [torch.rand(q_local, device="cuda", generator=g).add(0.5).bfloat16() for _ in range(world)]
        wk = [torch.rand(k_local, device="cuda", generator=g).add(0.5).bfloat16() for _ in range(world)]
        rq, rk = reference_qknorm(q, k, wq, wk, 1e-6)
        op(q, k, wq, wk)
        ctx.check_status()
        for r in range(world):
            assert torch.allclose(q[r].float(), rq[r], atol=3e-2, rtol=3e-2)
            assert torch.allclose(k[r].float(), rk[r], atol=3e-2, rtol=3e-2)


def test_put_signal_then_wait_get(native_lib):
    from commbench_b200.ops import shmem

    src = torch.randn(1 << 20, device="cuda")
    remote = torch.zeros_like(src)          # stands for the peer's copy
    sig = torch.zeros(4, dtype=torch.int32, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    shmem.put_signal(remote.data_ptr(), src, sig.data_ptr(), value=7)
    out = torch.empty_like(src)
    shmem.wait_get(sig.data_ptr(), 7, dst=out, src_ptr=remote.data_ptr(), status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and int(sig[0].item()) == 7
    assert torch.equal(out, src) and torch.equal(remote, src)
    # additive signal, as counters use it
    shmem.put_signal(remote.data_ptr(), src, sig.data_ptr() + 4, value=3, add=True)
    shmem.put_signal(remote.data_ptr(), src, sig.data_ptr() + 4, value=3, add=True)
    shmem.wait_get(sig.data_ptr() + 4, 6, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and int(sig[1].item()) == 6


def test_wait_for_a_signal_nobody_sends_times_out(native_lib):
    from commbench_b200.ops import shmem

    sig = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    shmem.wait_get(sig.data_ptr(), 1, timeout_s=0.05, status=st)
    torch.cuda.synchronize()
    assert (int(st.item()) >> 24) & 0xFF == 1        # CB_TIMEOUT_PEER_FLAG


def test_atomic_fetch_inc_tickets_are_consecutive(native_lib):
    from commbench_b200.ops import shmem

    counter = torch.zeros(1, dtype=torch.int64, device="cuda")
    t1, _ = shmem.atomic_fetch_inc(counter.data_ptr(), 100)
    t2, _ = shmem.atomic_fetch_inc(counter.data_ptr(), 50)
    torch.cuda.synchronize()
    assert t1.tolist() == list(range(100)) and t2.tolist() == list(range(100, 150))
    assert int(counter.item()) == 150


@pytest.mark.parametrize("side", [128, 512])
def test_tile_put_and_consume(native_lib, side):
    from commbench_b200.ops import shmem

    src = torch.randn(side, side, device="cuda")
    remote = torch.zeros_like(src)
    nt = (side // 64) ** 2
    flags = torch.zeros(nt, dtype=torch.int32, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    shmem.tile_put(remote.data_ptr(), src, 64, flags.data_ptr(), value=1)
    part = shmem.tile_consume(remote, 64, flags.data_ptr(), value=1, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    ref = src.view(side // 64, 64, side // 64, 64).sum(dim=(1, 3)).reshape(-1)
    assert torch.allclose(part, ref, atol=1e-2, rtol=1e-4)
