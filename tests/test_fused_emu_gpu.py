"""Fused GEMM+collective kernels with virtual ranks on ONE GPU (one cooperative launch),
against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(shape, seed, scale=0.25):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=g) * scale).bfloat16()


def _close(out, ref, tol=1.5e-2):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, f"max abs err {err} vs scale {scale}"


# bn 512 = a CTA pair (cluster of two) per 256 x 256 tile.
@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("bn", [512, 256, 128])
def test_emu_ag_gemm(native_lib, world, bn):
    from commbench_b200.ops.tp import AgGemm
    from commbench_b200.runtime.context import EmuContext

    Ml, K, Nn = 256, 512, 384
    ctx = EmuContext(world)
    op = AgGemm(ctx, max_m=Ml * world, k=K)
    a = [_rand((Ml, K), 10 + r) for r in range(world)]
    b = [_rand((Nn, K), 50 + r) for r in range(world)]
    full = torch.cat(a, dim=0).float()
    for it in range(3):   # three calls: both buffer parities and the flag reset are exercised
        outs = op(a, b, bn=bn)
        ctx.check_status()
        for r in range(world):
            _close(outs[r], full @ b[r].float().t())


@pytest.mark.parametrize("world", [2, 4])
def test_emu_gemm_rs(native_lib, world):
    from commbench_b200.ops.tp import GemmRs
    from commbench_b200.runtime.context import EmuContext

    M, K, Nn = 256 * world, 256, 384
    ctx = EmuContext(world)
    op = GemmRs(ctx, max_m=M, max_n=Nn)
    a = [_rand((M, K), 100 + r) for r in range(world)]
    b = [_rand((Nn, K), 200 + r) for r in range(world)]
    total = sum(a[r].float() @ b[r].float().t() for r in range(world))
    Ml = M // world
    for it in range(4):
        outs = op(a, b, bn=(256, 128, 512, 512)[it])
        ctx.check_status()
        for r in range(world):
            _close(outs[r], total[r * Ml:(r + 1) * Ml])


@pytest.mark.parametrize("bn", [512, 256])
def test_emu_gemm_rs_many_tiles_per_owner(native_lib, bn):
    """Several row and column blocks per owner, so that remote partials of a tile arrive
    while other tiles are in flight, over six calls (both parities, counters cleared)."""
    from commbench_b200.ops.tp import GemmRs
    from commbench_b200.runtime.context import EmuContext

    world = 2
    M, K, Nn = 1024 * world, 192, 1024 + 64
    ctx = EmuContext(world)
    op = GemmRs(ctx, max_m=M, max_n=Nn)
    a = [_rand((M, K), 500 + r) for r in range(world)]
    b = [_rand((Nn, K), 600 + r) for r in range(world)]
    total = sum(a[r].float() @ b[r].float().t() for r in range(world))
    Ml = M // world
    for it in range(6):
        outs = op(a, b, bn=bn)
        ctx.check_status()
        for r in range(world):
            _close(outs[r], total[r * Ml:(r + 1) * Ml])


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("oneshot", [True, False])
@pytest.mark.parametrize("M", [16, 200, 512])
def test_emu_gemm_ar(native_lib, world, oneshot, M):
    from commbench_b200.ops.tp import GemmAr
    from commbench_b200.runtime.context import EmuContext

    K, Nn = 256, 1024
    ctx = EmuContext(world)
    op = GemmAr(ctx, max_m=512, max_n=Nn)
    a = [_rand((M, K), 300 + r) for r in range(world)]
    b = [_rand((Nn, K), 400 + r) for r in range(world)]
    total = sum(a[r].float() @ b[r].float().t() for r in range(world))
    for it in range(3):
        outs = op(a, b, oneshot=oneshot, bn=64 if it < 2 else 128)
        ctx.check_status()
        for r in range(world):
            _close(outs[r], total)
        for r in range(1, world):
            assert torch.equal(outs[r], outs[0])


def test_tp_mlp_end_to_end_pipelined_matches_single_shot(native_lib):
    """One rank: tokens in pinned host memory, copied in four row chunks on a copy stream while
    the first GEMM of the earlier chunks runs; the metric equals the single-shot forward's, for
    the tcgen05 path and for the cuBLAS path."""
    from commbench_b200.models.tp_mlp import TPMLP
    from commbench_b200.runtime.context import CommContext

    ctx = CommContext(heap_bytes=64 << 20)
    mlp = TPMLP(ctx, hidden=512, intermediate=1024, max_tokens=8192, seed=2)
    assert mlp.host_chunks(8192) == 4 and mlp.host_chunks(1000) == 1
    xh = (torch.randn(8192, 512, generator=torch.Generator().manual_seed(1)) * 0.5).bfloat16().pin_memory()
    want = mlp.forward(xh.cuda()).float().abs().mean().item()
    for _ in range(3):                                   # repeated steps reuse the staging buffer
        got = mlp.forward_host(xh, fused=True)
        assert abs(got - want) <= 1e-3 * abs(want)
    got_u = mlp.forward_host(xh, fused=False)
    assert abs(got_u - want) <= 2e-2 * abs(want)
    ctx.check_status()
    ctx.close()


@pytest.mark.parametrize("kernel_first", [False, True])
def test_ag_gemm_consumes_rows_as_a_host_copy_delivers_them(native_lib, kernel_first):
    """The AG->GEMM kernel gated on per-256-row "has landed" words that a copy stream publishes
    with stream memory operations after each piece of a host-to-device copy.  With
    ``kernel_first`` the kernel is already running (and waiting, bounded) when the copies are
    enqueued: it must pick the rows up as they arrive and give the exact product."""
    from commbench_b200.ops.tp import AgGemm, stream_write_u32
    from commbench_b200.runtime.context import CommContext

    ctx = CommContext(heap_bytes=128 << 20)
    M, K, Nn, g = 2048, 1024, 768, 256
    op = AgGemm(ctx, max_m=M, k=K)
    gen = torch.Generator().manual_seed(5)
    a_host = (torch.randn(M, K, generator=gen) * 0.25).bfloat16().pin_memory()
    b = _rand((Nn, K), 6)
    a_dev = torch.zeros(M, K, device="cuda", dtype=torch.bfloat16)
    ready = torch.zeros(M // g, device="cuda", dtype=torch.int32)
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    for seq in (1, 2):                                   # a second step reuses buffers and words
        a_dev.zero_()
        torch.cuda.synchronize()

        def copies():
            with torch.cuda.stream(side):
                for c in range(M // g):
                    a_dev[c * g:(c + 1) * g].copy_(a_host[c * g:(c + 1) * g], non_blocking=True)
                    stream_write_u32(ready[c:c + 1], seq, side)

        if not kernel_first:
            copies()
        out = op(a_dev, b, src_ready=(ready, seq, g))
        if kernel_first:
            copies()
        torch.cuda.synchronize()
        ctx.check_status()
        ref = a_host.cuda().float() @ b.float().t()
        assert ((out.float() - ref).abs().max() / ref.abs().max()).item() < 2e-2
    ctx.close()
