"""tcgen05 GEMM vs a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, alpha=1.0):
    return alpha * (a.float() @ b.float().t())


def _check(out, ref, tol):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, f"max abs err {err} vs scale {scale}"


# bn 512 / 384 = a CTA pair (cluster of two, `tcgen05.mma.cta_group::2`) per 256 x 256 /
# 256 x 128 tile; the others one CTA per 128 x bn tile.
@pytest.mark.parametrize("bn", [512, 384, 256, 128, 64])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (384, 768, 1024),
                                   (1000, 1304, 520), (16, 8192, 1024)])
def test_gemm_bf16_matches_fp32_reference(native_lib, shape, bn):
    from commbench_b200.ops.gemm import gemm

    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(1234 + M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).mul_(0.5).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).mul_(0.5).bfloat16()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = gemm(a, b, bn=bn, status_ptr=status.data_ptr())
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0, hex(int(status[0].item()) & 0xffffffff)
    _check(out, _ref(a, b), 1e-2)


def test_gemm_pair_every_element_exact_on_small_ints(native_lib):
    """CTA-pair tiles: integer-valued inputs make fp32 accumulation exact, so a row or column
    half that lands in the wrong place shows up as a mismatch, not as noise."""
    from commbench_b200.ops.gemm import gemm

    M, N, K = 768, 1024, 320
    g = torch.Generator(device="cuda").manual_seed(11)
    a = torch.randint(-3, 4, (M, K), device="cuda", generator=g).bfloat16()
    b = torch.randint(-3, 4, (N, K), device="cuda", generator=g).bfloat16()
    for bn in (512, 384):
        out = gemm(a, b, bn=bn)
        assert torch.equal(out.float(), _ref(a, b).bfloat16().float()), bn


def test_gemm_bf16_full_tensor_exact_on_small_ints(native_lib):
    """Integer-valued inputs make the fp32 accumulation exact: every element must match."""
    from commbench_b200.ops.gemm import gemm

    M, N, K = 256, 512, 192
    g = torch.Generator(device="cuda").manual_seed(7)
    a = torch.randint(-3, 4, (M, K), device="cuda", generator=g).bfloat16()
    b = torch.randint(-3, 4, (N, K), device="cuda", generator=g).bfloat16()
    out = gemm(a, b, bn=128)
    ref = _ref(a, b)
    assert torch.equal(out.float(), ref.bfloat16().float())


def test_gemm_bf16_large_auto_tile(native_lib):
    from commbench_b200.ops.gemm import gemm

    M, N, K = 4096, 4096, 2048
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(M, K, device="cuda", generator=g).mul_(0.1).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).mul_(0.1).bfloat16()
    out = gemm(a, b, alpha=0.5)
    _check(out, _ref(a, b, 0.5), 1e-2)


@pytest.mark.parametrize("shape", [(128, 256, 128), (512, 1024, 512), (300, 520, 1024)])
def test_gemm_fp8_matches_fp32_reference(native_lib, shape):
    from commbench_b200.ops.gemm import gemm

    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(99)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(N, K, device="cuda", generator=g).to(torch.float8_e4m3fn)
    out = gemm(a, b, alpha=0.25, bn=128)
    _check(out, _ref(a, b, 0.25), 1e-2)
    out2 = gemm(a, b, alpha=0.25, bn=512)  # CTA pair
    _check(out2, _ref(a, b, 0.25), 1e-2)


def test_blockscaled_fp8_roundtrip_and_gemm(native_lib):
    """1x128 activation scales and 128x128 weight scales: quantise, check against a PyTorch
    emulation of the same scheme, then run the GEMM on the expanded operands."""
    from commbench_b200.ops.gemm import (dequantize_blockscaled, quantize_blockscaled)
    from commbench_b200.ops.gemm import gemm_fp8_blockscaled_expanded as gemm_fp8_blockscaled

    M, N, K = 256, 384, 512
    g = torch.Generator(device="cuda").manual_seed(21)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
    aq, as_ = quantize_blockscaled(a, 1)
    bq, bs = quantize_blockscaled(b, 128)
    # reference quantisation
    af = a.float().view(M, K // 128, 128)
    ref_s = af.abs().amax(-1) / 448.0
    assert torch.allclose(as_, ref_s, rtol=1e-6)
    bf = b.float().view(N // 128, 128, K // 128, 128)
    ref_bs = bf.abs().amax(dim=(1, 3)) / 448.0
    assert torch.allclose(bs, ref_bs, rtol=1e-6)
    ad = dequantize_blockscaled(aq, as_, 1)
    bd = dequantize_blockscaled(bq, bs, 128)
    assert (ad.float() - a.float()).abs().max() <= 0.07 * a.float().abs().max()
    out = gemm_fp8_blockscaled(aq, as_, bq, bs)
    ref = ad.float() @ bd.float().t()
    _check(out, ref, 1e-2)
    _check(out, a.float() @ b.float().t(), 6e-2)


def _bs_reference(aq, as_, bq, bs):
    """fp32 product of the SAME quantised operands with their block scales applied."""
    M, K = aq.shape
    N = bq.shape[0]
    a = aq.float().view(M, K // 128, 128) * as_[:, :, None]
    bsr = bs.repeat_interleave(128, dim=0)[:N]
    b = bq.float().view(N, K // 128, 128) * bsr[:, :, None]
    return a.view(M, K) @ b.view(N, K).t()


@pytest.mark.parametrize("pair", [True, False])
@pytest.mark.parametrize("shape", [(128, 256, 128), (256, 256, 256), (512, 768, 1024),
                                   (1000, 1304, 640), (256, 512, 4096)])
def test_blockscaled_fp8_gemm_in_kernel_scales(native_lib, shape, pair):
    """Block-scaled fp8 contraction with the scales applied inside the kernel (per K block,
    fp32 promotion): against the fp32 product of the same quantised operands."""
    from commbench_b200.ops.gemm import gemm_fp8_blockscaled, quantize_blockscaled

    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(5 + M + N + K)
    # magnitudes that differ per block, so that a wrong or missing scale shows
    a = torch.randn(M, K, device="cuda", generator=g) * \
        (1.0 + torch.arange(K // 128, device="cuda").float().repeat_interleave(128))[None, :]
    b = torch.randn(N, K, device="cuda", generator=g) * 0.02 * \
        (1.0 + (torch.arange(N, device="cuda") // 128).float())[:, None]
    aq, as_ = quantize_blockscaled(a.bfloat16().contiguous(), 1)
    bq, bs = quantize_blockscaled(b.bfloat16().contiguous(), 128)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = gemm_fp8_blockscaled(aq, as_, bq, bs, pair=pair, status_ptr=status.data_ptr())
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0, hex(int(status[0].item()) & 0xffffffff)
    ref = _bs_reference(aq, as_, bq, bs)
    _check(out, ref, 1e-2)
    _check(out, a.bfloat16().float() @ b.bfloat16().float().t(), 6e-2)


def test_pow2_quantisation_bytes_match_scales(native_lib):
    from commbench_b200.ops.gemm import quantize_blockscaled_pow2, sf_exponents

    g = torch.Generator(device="cuda").manual_seed(3)
    x = (torch.randn(300, 640, device="cuda", generator=g) * 3).bfloat16()
    for rb in (1, 128):
        q, s, sf = quantize_blockscaled_pow2(x, rb)
        assert sf.shape == (2, 300)
        assert torch.equal(torch.exp2(torch.log2(s).round()), s)          # powers of two
        per_row = s.repeat_interleave(rb, dim=0)[:300]
        assert torch.equal(torch.exp2(sf_exponents(sf, 5).float() - 127.0), per_row)
        assert bool((sf_exponents(sf, 8)[:, 5:] == 127).all())             # padding = 1.0
        amax = x.float().view(300, 5, 128).abs().amax(-1)
        if rb == 1:
            assert bool((s >= amax / 448.0).all()) and bool((s < 2 * amax / 448.0 + 1e-30).all())


@pytest.mark.parametrize("pair", [True, False])
@pytest.mark.parametrize("shape", [(128, 192, 128), (128, 192, 512), (256, 384, 1024),
                                   (1000, 1304, 640), (512, 8192, 2048)])
def test_fp8_gemm_with_hardware_block_scales(native_lib, shape, pair):
    """Power-of-two 1x128 / 128x128 block scales applied by the tensor core: against the fp32
    product of the same quantised operands with the same scales."""
    from commbench_b200.ops.gemm import gemm_fp8_mx, quantize_blockscaled_pow2

    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(9 + M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g) * \
        (1.0 + torch.arange(K // 128, device="cuda").float().repeat_interleave(128))[None, :] * \
        (1.0 + (torch.arange(M, device="cuda") % 7).float())[:, None]
    b = torch.randn(N, K, device="cuda", generator=g) * 0.02 * \
        (1.0 + (torch.arange(N, device="cuda") // 128).float())[:, None]
    aq, as_, asf = quantize_blockscaled_pow2(a.bfloat16().contiguous(), 1)
    bq, bs, bsf = quantize_blockscaled_pow2(b.bfloat16().contiguous(), 128)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = gemm_fp8_mx(aq, asf, bq, bsf, pair=pair, status_ptr=status.data_ptr())
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0, hex(int(status[0].item()) & 0xffffffff)
    ref = _bs_reference(aq, as_, bq, bs)
    _check(out, ref, 1e-2)
