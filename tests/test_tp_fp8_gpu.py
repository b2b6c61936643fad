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
