"""tcgen05 flash-attention forward and the exact merge of partial results, against a plain
PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _qkv(B, Sq, Skv, Hq, Hkv, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, Sq, Hq, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(B, Skv, Hkv, 128, device="cuda", generator=g).bfloat16()
    v = torch.randn(B, Skv, Hkv, 128, device="cuda", generator=g).bfloat16()
    return q, k, v


@pytest.mark.parametrize("impl", [1, 4])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [(1, 128, 128, 1, 1), (1, 256, 256, 4, 1), (2, 384, 384, 4, 2),
                                   (1, 200, 200, 2, 2), (1, 1024, 1024, 8, 2),
                                   (1, 2048, 2048, 4, 1)])
def test_flash_attention_matches_reference(native_lib, shape, causal, impl):
    from commbench_b200.ops.cp import flash_attention, reference_attention

    B, Sq, Skv, Hq, Hkv = shape
    q, k, v = _qkv(B, Sq, Skv, Hq, Hkv, 11 + Sq)
    o, lse = flash_attention(q, k, v, causal=causal, impl=impl)
    torch.cuda.synchronize()
    ro, rl = reference_attention(q, k, v, causal=causal)
    assert torch.allclose(o.float(), ro, atol=2e-2, rtol=2e-2), (o.float() - ro).abs().max()
    assert torch.allclose(lse, rl, atol=2e-2, rtol=1e-3)


def test_chunked_attention_with_offsets_merges_to_full(native_lib):
    """Keys split in three chunks (one entirely in the future of some queries); the merged
    result must equal attention over the whole sequence - the ring-attention invariant."""
    from commbench_b200.ops.cp import attn_merge, flash_attention, reference_attention

    B, S, Hq, Hkv = 1, 384, 4, 2
    q, k, v = _qkv(B, S, S, Hq, Hkv, 77)
    q_off = 128                      # queries are positions 128..511 of a longer sequence
    kfull = torch.cat([k, k.flip(1)], dim=1)[:, :640].contiguous()
    vfull = torch.cat([v, v.flip(1)], dim=1)[:, :640].contiguous()
    o_acc = torch.empty(B, S, Hq, 128, dtype=torch.float32, device="cuda")
    l_acc = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
    bounds = [(0, 256), (256, 512), (512, 640)]
    for i, (a, b) in enumerate(bounds):
        o, lse = flash_attention(q, kfull[:, a:b].contiguous(), vfull[:, a:b].contiguous(),
                                 causal=True, q_offset=q_off, kv_offset=a)
        attn_merge(o_acc, l_acc, o, lse, first=(i == 0))
    ro, rl = reference_attention(q, kfull, vfull, causal=True, q_offset=q_off, kv_offset=0)
    assert torch.allclose(o_acc, ro, atol=2e-2, rtol=2e-2)
    assert torch.allclose(l_acc, rl, atol=2e-2, rtol=1e-3)


def test_ring_and_ulysses_single_rank(native_lib):
    from commbench_b200.ops.cp import RingAttention, reference_attention, ulysses_attention
    from commbench_b200.runtime.context import CommContext

    ctx = CommContext(heap_bytes=64 << 20)
    q, k, v = _qkv(1, 256, 256, 4, 1, 5)
    ring = RingAttention(ctx, 1, 256, 4, 1)
    o, _ = ring.forward(q, k, v, causal=True)
    ro, _ = reference_attention(q, k, v, causal=True)
    assert torch.allclose(o.float(), ro, atol=2e-2, rtol=2e-2)
    o2 = ulysses_attention(ctx, q, k, v, causal=True)
    assert torch.allclose(o2.float(), ro, atol=2e-2, rtol=2e-2)
    ctx.check_status()
    ctx.close()
