"""Fused tensor-parallel GEMMs on block-scaled fp8 operands (virtual ranks on one GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(shape, seed, scale=0.25):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=g) * scale).bfloat16()


def _close(out, ref, tol):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, f"max abs err {err} vs scale {scale}"


@pytest.mark.parametrize("world", [2, 4])
def test_blockscaled_ag_gemm_and_gemm_rs(native_lib, world):
    from commbench_b200.ops.gemm import dequantize_blockscaled, quantize_blockscaled
    from commbench_b200.ops.tp import AgGemm, GemmRs
    from commbench_b200.ops.tp_fp8 import BlockScaledWeight, fused_blockscaled
    from commbench_b200.runtime.context import EmuContext

    Ml, K, Nn = 256, 512, 384
    ctx = EmuContext(world)
    # all-gather -> GEMM: activations sharded by rows, weights by output features
    a = [_rand((Ml, K), 10 + r, 1.0) for r in range(world)]
    w = [_rand((Nn, K), 50 + r, 0.05) for r in range(world)]
    aq = [quantize_blockscaled(x, 1) for x in a]
    wq = [BlockScaledWeight.from_bf16(x) for x in w]
    op = AgGemm(ctx, max_m=Ml * world, k=K)
    outs = fused_blockscaled(op, [q for q, _ in aq], [s for _, s in aq], wq)
    ctx.check_status()
    a_deq = torch.cat([dequantize_blockscaled(q, s, 1) for q, s in aq]).float()
    a_full = torch.cat(a).float()
    for r in range(world):
        _close(outs[r], a_deq @ wq[r].bf16().float().t(), 1.5e-2)       # exact up to bf16 output
        _close(outs[r], a_full @ w[r].float().t(), 8e-2)                # fp8 quantisation error
    assert wq[0].bf16() is wq[0].bf16()                                  # expansion is cached
    # GEMM -> reduce-scatter: K sharded
    M, Kl, N2 = 256 * world, 256, 512
    a2 = [_rand((M, Kl), 100 + r, 1.0) for r in range(world)]
    w2 = [_rand((N2, Kl), 150 + r, 0.05) for r in range(world)]
    a2q = [quantize_blockscaled(x, 1) for x in a2]
    w2q = [BlockScaledWeight.from_bf16(x) for x in w2]
    rs = GemmRs(ctx, M, N2)
    outs2 = fused_blockscaled(rs, [q for q, _ in a2q], [s for _, s in a2q], w2q)
    ctx.check_status()
    total = sum(dequantize_blockscaled(q, s, 1).float() @ w2q[r].bf16().float().t()
                for r, (q, s) in enumerate(a2q))
    rows = M // world
    for r in range(world):
        _close(outs2[r], total[r * rows:(r + 1) * rows], 2e-2)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("bn", [512, 256])
def test_per_tensor_fp8_fused_ops(native_lib, world, bn):
    """fp8 e4m3 tensors fed straight to the fused kernels (one scale per tensor folded into
    alpha), against the fp32 product of the same fp8 values."""
    from commbench_b200.ops.tp import AgGemm, GemmRs
    from commbench_b200.runtime.context import EmuContext

    f8 = torch.float8_e4m3fn
    Ml, K, Nn = 256, 512, 384
    ctx = EmuContext(world)
    a = [_rand((Ml, K), 10 + r, 1.0).to(f8) for r in range(world)]
    w = [_rand((Nn, K), 50 + r, 1.0).to(f8) for r in range(world)]
    op = AgGemm(ctx, max_m=Ml * world, k=K, dtype=f8)
    full = torch.cat([x.float() for x in a])
    for it in range(3):
        outs = op(a, w, alpha=0.125, bn=bn)
        ctx.check_status()
        for r in range(world):
            _close(outs[r], 0.125 * (full @ w[r].float().t()), 1e-2)
    M, Kl, N2 = 256 * world, 256, 512
    a2 = [_rand((M, Kl), 100 + r, 1.0).to(f8) for r in range(world)]
    w2 = [_rand((N2, Kl), 150 + r, 1.0).to(f8) for r in range(world)]
    rs = GemmRs(ctx, M, N2)
    total = 0.25 * sum(a2[r].float() @ w2[r].float().t() for r in range(world))
    rows = M // world
    for it in range(3):
        outs2 = rs(a2, w2, alpha=0.25, bn=bn)
        ctx.check_status()
        for r in range(world):
            _close(outs2[r], total[r * rows:(r + 1) * rows], 1.5e-2)


def _bs_ref(q, s, rb):
    rows, K = q.shape
    sr = s.repeat_interleave(rb, dim=0)[:rows]
    return (q.float().view(rows, K // 128, 128) * sr[:, :, None]).view(rows, K)


@pytest.mark.parametrize("world", [2, 4])
def test_hardware_blockscaled_fused_ops(native_lib, world):
    """fp8 operands with power-of-two 1x128 / 128x128 block scales applied by the tensor cores
    inside the fused kernels; the gathered rows' scale words travel with the rows.  Against the
    fp32 product of the same quantised operands with the same scales."""
    from commbench_b200.ops.gemm import quantize_blockscaled_pow2
    from commbench_b200.ops.tp import AgGemm, GemmRs
    from commbench_b200.runtime.context import EmuContext

    f8 = torch.float8_e4m3fn
    Ml, K, Nn = 512, 1024, 384
    ctx = EmuContext(world)
    kscale = (1.0 + torch.arange(K // 128, device="cuda").float().repeat_interleave(128))[None, :]
    a = [(_rand((Ml, K), 10 + r, 1.0).float() * kscale * (1 + r)).bfloat16() for r in range(world)]
    w = [(_rand((Nn, K), 50 + r, 0.05).float() *
          (1.0 + (torch.arange(Nn, device="cuda") // 128).float())[:, None]).bfloat16()
         for r in range(world)]
    aq = [quantize_blockscaled_pow2(x, 1) for x in a]
    wq = [quantize_blockscaled_pow2(x, 128) for x in w]
    op = AgGemm(ctx, max_m=Ml * world, k=K, dtype=f8)
    a_ref = torch.cat([_bs_ref(q, s, 1) for q, s, _ in aq])
    for it in range(3):
        outs = op([q for q, _, _ in aq], [q for q, _, _ in wq],
                  a_sf=[f for _, _, f in aq], b_sf=[f for _, _, f in wq])
        ctx.check_status()
        for r in range(world):
            _close(outs[r], a_ref @ _bs_ref(wq[r][0], wq[r][1], 128).t(), 1.5e-2)
    M, Kl, N2 = 256 * world, 512, 576
    a2 = [(_rand((M, Kl), 100 + r, 1.0).float() * (1 + (torch.arange(M, device="cuda") % 5).float())[:, None]).bfloat16()
          for r in range(world)]
    w2 = [_rand((N2, Kl), 150 + r, 0.05) for r in range(world)]
    a2q = [quantize_blockscaled_pow2(x, 1) for x in a2]
    w2q = [quantize_blockscaled_pow2(x, 128) for x in w2]
    rs = GemmRs(ctx, M, N2)
    total = sum(_bs_ref(a2q[r][0], a2q[r][1], 1) @ _bs_ref(w2q[r][0], w2q[r][1], 128).t()
                for r in range(world))
    rows = M // world
    for it in range(3):
        outs2 = rs([q for q, _, _ in a2q], [q for q, _, _ in w2q],
                   a_sf=[f for _, _, f in a2q], b_sf=[f for _, _, f in w2q])
        ctx.check_status()
        for r in range(world):
            _close(outs2[r], total[r * rows:(r + 1) * rows], 2e-2)
