"""MoE kernels: router, layout, and the whole expert-parallel layer with virtual ranks on one
GPU, against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_router_topk_matches_torch(native_lib):
    from commbench_b200.ops.moe import router_topk

    g = torch.Generator(device="cuda").manual_seed(5)
    logits = torch.randn(777, 256, device="cuda", generator=g)
    idx, w = router_topk(logits, 8)
    p = torch.softmax(logits, dim=-1)
    tw, ti = torch.topk(p, 8, dim=-1)
    tw = tw / tw.sum(-1, keepdim=True)
    assert torch.equal(idx.long(), ti)
    assert torch.allclose(w, tw, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("T,K,R", [(257, 1, 1), (1024, 2, 2), (4096, 8, 8), (4097, 4, 4)])
def test_dispatch_layout_matches_cpu_reference(native_lib, T, K, R):
    from commbench_b200.ops.moe import dispatch_layout

    E = 32
    g = torch.Generator(device="cuda").manual_seed(T + K)
    # k distinct experts per token; some patterns put several experts on the same rank
    idx = torch.rand(T, E, device="cuda", generator=g).argsort(dim=1)[:, :K].int()
    idx[::7, 0] = -1                      # masked selections are skipped
    per_e, per_r, in_r = dispatch_layout(idx, R, E)
    ci = idx.cpu()
    ref_e = torch.zeros(E, dtype=torch.int32)
    ref_in = torch.zeros(T, R, dtype=torch.bool)
    for k in range(K):
        col = ci[:, k]
        ok = col >= 0
        ref_e += torch.bincount(col[ok].long(), minlength=E).int()
        ref_in[ok.nonzero().squeeze(1), (col[ok] // (E // R)).long()] = True
    assert torch.equal(per_e.cpu(), ref_e)
    assert torch.equal(in_r.cpu(), ref_in)
    assert torch.equal(per_r.cpu(), ref_in.sum(0).int())


@pytest.mark.parametrize("dispatch", ["per_pair", "per_token"])
@pytest.mark.parametrize("fused_swiglu", [True, False])
@pytest.mark.parametrize("world", [1, 2, 4])
def test_moe_layer_virtual_ranks(native_lib, world, fused_swiglu, dispatch):
    from commbench_b200.ops.moe import MoELayer, reference_moe, router_topk
    from commbench_b200.runtime.context import EmuContext

    T, H, I, E, K = 96, 512, 256, 8, 2
    ctx = EmuContext(world)
    layer = MoELayer(ctx, T, H, I, E, K, capacity_factor=float(world) * 2,
                     fused_swiglu=fused_swiglu, dispatch=dispatch)
    assert layer.launches_per_call == (8 if fused_swiglu else 10)
    xs, idxs, ws = [], [], []
    for r in range(world):
        g = torch.Generator(device="cuda").manual_seed(100 + r)
        xs.append(torch.randn(T, H, device="cuda", generator=g).bfloat16())
        i, w = router_topk(torch.randn(T, E, device="cuda", generator=g), K)
        idxs.append(i)
        ws.append(w)
    w1_all = torch.cat([layer.weights(r)[0] for r in range(world)])
    w2_all = torch.cat([layer.weights(r)[1] for r in range(world)])
    for it in range(2):     # second call: counters and flags were reset by the first
        ys = layer.forward(xs, idxs, ws)
        ctx.check_status()
        for r in range(world):
            ref = reference_moe(xs[r], idxs[r], ws[r], w1_all, w2_all, I)
            err = (ys[r].float() - ref).abs().max().item()
            scale = ref.abs().max().item() + 1e-6
            assert err / scale < 3e-2, (it, r, err, scale)
        # the receive kernel re-armed its own counters (no fill launch between two calls)
        for st in layer.states:
            assert int(layer._local(layer.arrived, st).view(torch.int32).abs().sum()) == 0
            assert int(st.recv_ctas.abs().sum()) == 0
            assert int(layer._local(layer.done, st).view(torch.int32).abs().sum()) == 0
    # the two optional bias inputs of the combine reduction (shared expert / residual)
    b0 = [torch.randn(T, H, device="cuda").bfloat16() for _ in range(world)]
    b1 = [torch.randn(T, H, device="cuda").bfloat16() for _ in range(world)]
    ys = layer.forward(xs, idxs, ws, bias0=b0, bias1=b1)
    ctx.check_status()
    for r in range(world):
        ref = reference_moe(xs[r], idxs[r], ws[r], w1_all, w2_all, I) + b0[r].float() + b1[r].float()
        err = (ys[r].float() - ref).abs().max().item()
        assert err / (ref.abs().max().item() + 1e-6) < 3e-2, (r, err)


@pytest.mark.parametrize("n,E", [(100, 4), (4096 * 8, 256), (777, 33)])
def test_expert_sort_is_a_stable_sort(native_lib, n, E):
    from commbench_b200.ops.moe import expert_sort

    g = torch.Generator(device="cuda").manual_seed(n)
    idx = torch.randint(0, E, (n,), device="cuda", generator=g, dtype=torch.int32)
    idx[::11] = -1
    sp, counts = expert_sort(idx, E)
    valid = (idx >= 0).nonzero().squeeze(1)
    order = valid[torch.sort(idx[valid].long(), stable=True).indices]
    assert torch.equal(sp[:order.numel()].long(), order)
    assert bool((sp[order.numel():] == -1).all())
    assert torch.equal(counts.long(), torch.bincount(idx[valid].long(), minlength=E))
