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
    q, k, v = _qkv(1, 512, 512, 4, 1, 5)
    ring = RingAttention(ctx, 1, 512, 4, 1)
    o, lse = ring.forward(q, k, v, causal=True)
    ro, rl = reference_attention(q, k, v, causal=True)
    assert torch.allclose(o.float(), ro, atol=2e-2, rtol=2e-2)
    assert torch.allclose(lse, rl, atol=2e-2, rtol=1e-3)
    o2 = ulysses_attention(ctx, q, k, v, causal=True)
    assert torch.allclose(o2.float(), ro, atol=2e-2, rtol=2e-2)
    ctx.check_status()
    ctx.close()


def _full(B, S, Hq, Hkv, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, S, Hq, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(B, S, Hkv, 128, device="cuda", generator=g).bfloat16()
    v = torch.randn(B, S, Hkv, 128, device="cuda", generator=g).bfloat16()
    return q, k, v


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("zigzag", [True, False])
@pytest.mark.parametrize("causal", [True, False])
def test_ring_attention_kernel_virtual_ranks(native_lib, world, zigzag, causal):
    """W virtual ranks on one GPU (their launches pull from each other's buffers, none waits
    for another): every rank's rows must equal full-sequence attention, over three calls."""
    from commbench_b200.ops.cp import RingAttention, reference_attention, zigzag_shard
    from commbench_b200.runtime.context import EmuContext

    B, Sl, Hq, Hkv = 2, 512, 4, 2
    S = Sl * world
    q, k, v = _full(B, S, Hq, Hkv, 31 + world)
    ro, rl = reference_attention(q, k, v, causal=causal)
    if zigzag:
        shard = lambda x, r: zigzag_shard(x, world, r)
    else:
        shard = lambda x, r: x[:, r * Sl:(r + 1) * Sl].contiguous()
    ctx = EmuContext(world)
    ring = RingAttention(ctx, B, Sl, Hq, Hkv, zigzag=zigzag, num_comm=2)
    qs = [shard(q, r) for r in range(world)]
    ks = [shard(k, r) for r in range(world)]
    vs = [shard(v, r) for r in range(world)]
    for it in range(3):
        outs, lses = ring.forward(qs, ks, vs, causal=causal)
        ctx.check_status()
        for r in range(world):
            assert torch.allclose(outs[r].float(), shard(ro, r), atol=2e-2, rtol=2e-2), (it, r)
            ref_l = shard(rl.permute(0, 2, 1), r).permute(0, 2, 1)
            assert torch.allclose(lses[r], ref_l, atol=2e-2, rtol=1e-3), (it, r)
    # the same object with the other mask: the list of pieces to pull changes
    ro2, _ = reference_attention(q, k, v, causal=not causal)
    for it in range(2):
        outs, _ = ring.forward(qs, ks, vs, causal=not causal)
        ctx.check_status()
        for r in range(world):
            assert torch.allclose(outs[r].float(), shard(ro2, r), atol=2e-2, rtol=2e-2), (it, r)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("causal", [True, False])
def test_ulysses_attention_kernel_virtual_ranks(native_lib, world, causal):
    """Sequence-sharded in and out; each virtual rank attends for its head slice over the whole
    sequence, reading Q from and writing O to the other ranks' tensors."""
    from commbench_b200.ops.cp import UlyssesAttention, reference_attention
    from commbench_b200.runtime.context import EmuContext

    B, Sl, Hq, Hkv = 1, 512, 8, 4
    S = Sl * world
    q, k, v = _full(B, S, Hq, Hkv, 57 + world)
    ro, _ = reference_attention(q, k, v, causal=causal)
    ctx = EmuContext(world)
    op = UlyssesAttention(ctx, B, Sl, Hq, Hkv, num_comm=2)
    sh = lambda x, r: x[:, r * Sl:(r + 1) * Sl].contiguous()
    for it in range(3):
        outs = op.forward([sh(q, r) for r in range(world)], [sh(k, r) for r in range(world)],
                          [sh(v, r) for r in range(world)], causal=causal)
        ctx.check_status()
        for r in range(world):
            assert torch.allclose(outs[r].float(), sh(ro, r), atol=2e-2, rtol=2e-2), (it, r)
