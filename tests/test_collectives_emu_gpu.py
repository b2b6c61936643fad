"""Collective kernels with W virtual ranks on ONE GPU (single cooperative launch per op),
checked against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(world, shape, dtype, seed=0):
    xs = []
    for r in range(world):
        g = torch.Generator(device="cuda").manual_seed(seed + r)
        xs.append((torch.rand(shape, device="cuda", generator=g) * 2 - 1).to(dtype))
    return xs


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "twoshot_push"])
@pytest.mark.parametrize("numel", [8, 1000, 4096, 262144 + 24])
def test_emu_all_reduce(native_lib, world, algo, numel):
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import EmuContext

    ctx = EmuContext(world)
    xs = _inputs(world, (numel,), torch.bfloat16)
    ref = sum(x.float() for x in xs)
    outs = coll.emu_all_reduce(ctx, xs, algo=algo)
    ctx.check_status()
    for o in outs:
        assert torch.allclose(o.float(), ref, atol=2e-2, rtol=2e-2)
    # every rank must hold the same bits
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    # a second call on the same context exercises the epoch counters
    outs2 = coll.emu_all_reduce(ctx, xs, algo=algo)
    ctx.check_status()
    assert torch.equal(outs2[0], outs[0])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_emu_all_reduce_dtypes(native_lib, dtype):
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import EmuContext

    ctx = EmuContext(4)
    xs = _inputs(4, (5000,), dtype)
    ref = sum(x.double() for x in xs)
    for algo in ("oneshot", "twoshot"):
        outs = coll.emu_all_reduce(ctx, xs, algo=algo)
        ctx.check_status()
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert torch.allclose(outs[2].double(), ref, atol=tol, rtol=tol)


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("push", [False, True])
def test_emu_all_gather(native_lib, world, push):
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import EmuContext

    ctx = EmuContext(world)
    xs = _inputs(world, (96, 40), torch.bfloat16)
    outs = coll.emu_all_gather(ctx, xs, push=push)
    ctx.check_status()
    ref = torch.cat(xs, dim=0)
    for o in outs:
        assert torch.equal(o, ref)


def test_emu_all_gather_unaligned_shard(native_lib):
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import EmuContext

    ctx = EmuContext(4)
    xs = _inputs(4, (7, 3), torch.bfloat16)   # 42 bytes per shard
    outs = coll.emu_all_gather(ctx, xs)
    ctx.check_status()
    assert torch.equal(outs[1], torch.cat(xs, dim=0))


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("unroll", [0, 1, 2, 8])
def test_emu_reduce_scatter(native_lib, world, unroll):
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import EmuContext

    ctx = EmuContext(world)
    xs = _inputs(world, (world * 64, 72), torch.bfloat16)
    outs = coll.emu_reduce_scatter(ctx, xs, unroll=unroll)
    ctx.check_status()
    total = sum(x.float() for x in xs)
    for r, o in enumerate(outs):
        assert torch.allclose(o.float(), total[r * 64:(r + 1) * 64], atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("push,unroll", [(False, 0), (False, 8), (True, 0), (True, 2)])
def test_emu_all_to_all_flat(native_lib, world, push, unroll):
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import EmuContext

    ctx = EmuContext(world)
    xs = _inputs(world, (world * 24, 64), torch.bfloat16)
    outs = coll.emu_all_to_all(ctx, xs, push=push, unroll=unroll)
    ctx.check_status()
    for r in range(world):
        ref = torch.cat([xs[p][r * 24:(r + 1) * 24] for p in range(world)], dim=0)
        assert torch.equal(outs[r], ref)


@pytest.mark.parametrize("world", [2, 4])
def test_emu_all_to_all_4d_roundtrip(native_lib, world):
    """Forward (sequence-sharded -> head-sharded) against an index-level reference, then the
    inverse must recover the input (the reference's forward+inverse recovery check)."""
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import EmuContext

    ctx = EmuContext(world)
    B, Sl, H, D = 2, 12, 8, 64
    xs = _inputs(world, (B, Sl, H, D), torch.bfloat16)
    outs = coll.emu_all_to_all_4d(ctx, xs, to_heads=True)
    ctx.check_status()
    Hl = H // world
    full = torch.cat(xs, dim=1)                       # [B, S, H, D]
    for r in range(world):
        assert torch.equal(outs[r], full[:, :, r * Hl:(r + 1) * Hl, :].contiguous())
    back = coll.emu_all_to_all_4d(ctx, outs, to_heads=False)
    ctx.check_status()
    for r in range(world):
        assert torch.equal(back[r], xs[r])


def test_emu_broadcast_and_barrier(native_lib):
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import EmuContext

    ctx = EmuContext(4)
    xs = _inputs(4, (1001,), torch.float32)
    want = xs[2].clone()
    coll.emu_broadcast(ctx, xs, root=2)
    ctx.check_status()
    for x in xs:
        assert torch.equal(x, want)
    coll.emu_barrier(ctx, iters=10)
    ctx.check_status()


def test_wait_times_out_and_reports_status(native_lib):
    """A flag that nothing sets: the bounded wait must run out, the kernel must return and
    leave a status word, and the context must stay usable."""
    import ctypes as C

    from commbench_b200 import _native as N
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import CommError, EmuContext

    ctx = EmuContext(2, timeout_s=0.05)
    # Virtual rank 0 alone: its peer never signals because the grid has one slice only.
    args = [coll._fill_args(ctx.comms[0], [], 0, 0, 0, 0)]
    table = ctx.args_table(args)
    rc = ctx.lib.cb_barrier_launch(C.byref(args[0]), C.c_void_p(table.data_ptr()), 1, 1, 0,
                                   N.stream_ptr())
    assert rc == 0
    with pytest.raises(CommError, match="timeout"):
        ctx.check_status()
    # the device and context still work
    ctx2 = EmuContext(2)
    xs = _inputs(2, (64,), torch.bfloat16)
    outs = coll.emu_all_reduce(ctx2, xs)
    ctx2.check_status()
    assert torch.allclose(outs[0].float(), xs[0].float() + xs[1].float(), atol=2e-2)


@pytest.mark.parametrize("world", [2, 8])
def test_collectives_are_bit_stable_under_start_jitter(native_lib, world, monkeypatch):
    """Debug stress: every CTA starts after its own pseudo-random delay (up to 200 us).  Results
    must be bit-identical to the run without delays, call after call."""
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import EmuContext

    xs = _inputs(world, (world * 4096 + world * 8,), torch.bfloat16, seed=11)
    calm = EmuContext(world)
    want_ar = coll.emu_all_reduce(calm, xs, algo="twoshot")[0].clone()
    want_rs = [o.clone() for o in coll.emu_reduce_scatter(calm, xs)]
    want_a2a = [o.clone() for o in coll.emu_all_to_all(calm, xs)]
    calm.check_status()
    monkeypatch.setenv("CB200_DEBUG_JITTER_NS", "200000")
    ctx = EmuContext(world)
    assert ctx.comms[0].jitter_ns == 200000
    for _ in range(3):
        for o in coll.emu_all_reduce(ctx, xs, algo="twoshot"):
            assert torch.equal(o, want_ar)
        for o, w in zip(coll.emu_reduce_scatter(ctx, xs), want_rs):
            assert torch.equal(o, w)
        for o, w in zip(coll.emu_all_to_all(ctx, xs), want_a2a):
            assert torch.equal(o, w)
        gathered = coll.emu_all_gather(ctx, xs, push=True)
        assert torch.equal(gathered[world - 1], torch.cat(xs))
        ctx.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("algo", ["twoshot", "twoshot_push"])
@pytest.mark.parametrize("unroll", [1, 2, 4, 8])
def test_emu_all_reduce_vectors_in_flight(native_lib, world, algo, unroll):
    """Every unroll depth of the pull loops gives the same bits as the default one, on a size
    with full iterations, a remainder and a ragged tail."""
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import EmuContext

    ctx = EmuContext(world)
    xs = _inputs(world, (3 * 512 * 8 * 8 + 44,), torch.bfloat16)
    base = coll.emu_all_reduce(ctx, xs, algo="twoshot", blocks=2)
    outs = coll.emu_all_reduce(ctx, xs, algo=algo, blocks=2, unroll=unroll)
    ctx.check_status()
    for o in outs:
        assert torch.equal(o, base[0])


@pytest.mark.gpu
@pytest.mark.parametrize("unroll", [2, 4, 8])
def test_emu_all_gather_vectors_in_flight(native_lib, unroll):
    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime.context import EmuContext

    ctx = EmuContext(4)
    xs = _inputs(4, (5 * 512 * 8 + 64,), torch.bfloat16)
    ref = torch.cat(xs)
    for push in (False, True):
        outs = coll.emu_all_gather(ctx, xs, push=push, unroll=unroll, blocks=1)
        ctx.check_status()
        for o in outs:
            assert torch.equal(o.flatten(), ref)
