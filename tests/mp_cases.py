"""Multi-process checks run under torch.distributed.run (one rank per GPU).

Prints one JSON line per check from rank 0 ("check", "ok", "detail") and exits non-zero
if any check failed on any rank.  Usage: torchrun ... tests/mp_cases.py [group ...]
with groups out of moe, attention, p2p, parallel, all_reduce, all_gather, reduce_scatter,
all_to_all, broadcast, ag_gemm, gemm_rs, gemm_ar (none named: all of them) and, only when
named, moe_per_token (the layer with one dispatch row per token and rank).
"""
import json
import os
import sys
import traceback

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

RESULTS = []


def report(name, ok, detail=""):
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ok_all = bool(flag.item())
    RESULTS.append(ok_all)
    if dist.get_rank() == 0:
        print(json.dumps({"check": name, "ok": ok_all, "detail": str(detail)[:300]}), flush=True)


def guarded(name):
    def deco(fn):
        def run(*a, **k):
            try:
                fn(*a, **k)
            except Exception as e:  # noqa: BLE001
                traceback.print_exc()
                report(name, False, repr(e))
        return run
    return deco


def uniform(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.rand(shape, device="cuda", generator=g) * 2 - 1).to(dtype)


def gather_all(x):
    outs = [torch.empty_like(x) for _ in range(dist.get_world_size())]
    dist.all_gather(outs, x)
    return outs


def main():
    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    from commbench_b200.ops import collectives as coll
    from commbench_b200.ops.tp import AgGemm, GemmAr, GemmRs
    from commbench_b200.runtime.context import CommContext

    ctx = CommContext(heap_bytes=1 << 30)
    report("context", True, f"mode={ctx.mode} multicast={ctx.has_multicast}")

    @guarded("all_reduce")
    def t_all_reduce():
        algos = ["oneshot", "twoshot", "twoshot_push"] + (["nvls"] if ctx.has_multicast else [])
        for numel in (8, 2048, 1 << 16, (1 << 20) + 8, 1 << 24):
            x = uniform((numel,), rank)
            ref = sum(t.float() for t in gather_all(x))
            for algo in algos:
                y = coll.all_reduce(ctx, x.clone(), algo=algo)
                ctx.check_status()
                ok = torch.allclose(y.float(), ref, atol=5e-2, rtol=5e-2)
                report(f"all_reduce/{algo}/{numel}", ok, (y.float() - ref).abs().max().item())
        # symmetric, zero-copy, in place
        t, _ = ctx.empty((1 << 20,), torch.bfloat16)
        for algo in algos[1:]:
            t.copy_(uniform((1 << 20,), 100 + rank))
            ref = sum(u.float() for u in gather_all(t.clone()))
            torch.cuda.synchronize(); dist.barrier()
            coll.all_reduce(ctx, t, algo=algo)
            ctx.check_status()
            report(f"all_reduce/symmetric/{algo}", torch.allclose(t.float(), ref, atol=5e-2, rtol=5e-2))
        xf = uniform((4099,), 7 + rank, torch.float32)
        ref = sum(t.double() for t in gather_all(xf))
        y = coll.all_reduce(ctx, xf.clone(), algo="auto")
        ctx.check_status()
        report("all_reduce/fp32", torch.allclose(y.double(), ref, atol=1e-5, rtol=1e-5))
        # launch-shape knobs: every grid size and depth gives the same bits as the default
        t.copy_(uniform((1 << 20,), 300 + rank))
        keep = t.clone()
        torch.cuda.synchronize(); dist.barrier()
        base = coll.all_reduce(ctx, t, algo="twoshot").clone()
        same = True
        for algo, blocks, unroll in (("twoshot", 7, 2), ("twoshot_push", 32, 8), ("twoshot_push", 128, 1)):
            t.copy_(keep)
            torch.cuda.synchronize(); dist.barrier()
            same = same and torch.equal(coll.all_reduce(ctx, t, algo=algo, blocks=blocks, unroll=unroll), base)
            ctx.check_status()
        report("all_reduce/launch_shapes_bit_identical", same)

    @guarded("all_gather")
    def t_all_gather():
        x = uniform((300, 72), 20 + rank)
        ref = torch.cat(gather_all(x), dim=0)
        y = coll.all_gather(ctx, x)
        ctx.check_status()
        report("all_gather/pull", torch.equal(y, ref))
        out, _ = ctx.empty((300 * world, 72), torch.bfloat16)
        coll.all_gather(ctx, x, out=out)
        ctx.check_status()
        report("all_gather/push", torch.equal(out, ref))

    @guarded("reduce_scatter")
    def t_reduce_scatter():
        x = uniform((world * 128, 256), 30 + rank)
        total = sum(t.float() for t in gather_all(x))
        ref = total[rank * 128:(rank + 1) * 128]
        y = coll.reduce_scatter(ctx, x, use_nvls=False)
        ctx.check_status()
        report("reduce_scatter/pull", torch.allclose(y.float(), ref, atol=5e-2, rtol=5e-2))
        if ctx.has_multicast:
            y = coll.reduce_scatter(ctx, x, use_nvls=True)
            ctx.check_status()
            report("reduce_scatter/nvls", torch.allclose(y.float(), ref, atol=5e-2, rtol=5e-2))

    @guarded("all_to_all")
    def t_all_to_all():
        x = uniform((world * 64, 128), 40 + rank)
        ref = torch.empty_like(x)
        dist.all_to_all_single(ref, x)
        y = coll.all_to_all(ctx, x)
        ctx.check_status()
        report("all_to_all/flat", torch.equal(y, ref))
        y = coll.all_to_all(ctx, x, push=True, unroll=8)
        ctx.check_status()
        report("all_to_all/flat_push_staged", torch.equal(y, ref))
        so, _ = ctx.empty(tuple(x.shape), torch.bfloat16)
        coll.all_to_all(ctx, x, out=so)
        ctx.check_status()
        report("all_to_all/flat_push_symmetric_out", torch.equal(so, ref))
        B, Sl, H, D = 1, 96, 8 * world, 128
        q = uniform((B, Sl, H, D), 50 + rank)
        full = torch.cat(gather_all(q), dim=1)
        Hl = H // world
        y = coll.all_to_all_4d(ctx, q, to_heads=True)
        ctx.check_status()
        report("all_to_all/4d_fwd", torch.equal(y, full[:, :, rank * Hl:(rank + 1) * Hl].contiguous()))
        z = coll.all_to_all_4d(ctx, y, to_heads=False)
        ctx.check_status()
        report("all_to_all/4d_roundtrip", torch.equal(z, q))

    @guarded("broadcast")
    def t_broadcast():
        for root in (0, world - 1):
            x = uniform((5000,), 60 + rank, torch.float32)
            ref = x.clone()
            dist.broadcast(ref, src=root)
            coll.broadcast(ctx, x, root=root)
            ctx.check_status()
            report(f"broadcast/root{root}", torch.equal(x, ref))
        coll.barrier(ctx, iters=5)
        ctx.check_status()
        if ctx.has_multicast:
            coll.barrier(ctx, iters=5, use_nvls=True)
            ctx.check_status()
        report("barrier", True)

    def rnd(shape, seed, scale=0.25):
        g = torch.Generator(device="cuda").manual_seed(seed)
        return (torch.randn(shape, device="cuda", generator=g) * scale).bfloat16()

    def close(out, ref, tol=1.5e-2):
        return ((out.float() - ref).abs().max() / (ref.abs().max() + 1e-6)).item() < tol

    @guarded("ag_gemm")
    def t_ag_gemm():
        Ml, K, Nn = 512, 1024, 768
        op = AgGemm(ctx, max_m=Ml * world, k=K)
        a, b = rnd((Ml, K), 70 + rank), rnd((Nn, K), 80 + rank)
        ref = torch.cat(gather_all(a), dim=0).float() @ b.float().t()
        for it in range(4):
            c = op(a, b, bn=256 if it % 2 == 0 else 128)
            ctx.check_status()
            report(f"ag_gemm/{it}", close(c, ref))

    @guarded("gemm_rs")
    def t_gemm_rs():
        M, K, Nn = 256 * world, 512, 768
        op = GemmRs(ctx, max_m=M, max_n=Nn)
        a, b = rnd((M, K), 90 + rank), rnd((Nn, K), 95 + rank)
        part = (a.float() @ b.float().t())
        dist.all_reduce(part)
        Ml = M // world
        for it in range(4):
            o = op(a, b)
            ctx.check_status()
            report(f"gemm_rs/{it}", close(o, part[rank * Ml:(rank + 1) * Ml]))

    @guarded("gemm_ar")
    def t_gemm_ar():
        K, Nn = 512, 2048
        op = GemmAr(ctx, max_m=1024, max_n=Nn)
        for M in (16, 128, 1024):
            a, b = rnd((M, K), 110 + rank), rnd((Nn, K), 120 + rank)
            part = (a.float() @ b.float().t())
            dist.all_reduce(part)
            for oneshot in (True, False):
                for it in range(3):
                    o = op(a, b, oneshot=oneshot)
                    ctx.check_status()
                    report(f"gemm_ar/M{M}/oneshot{int(oneshot)}/{it}", close(o, part))
            for it in range(3):             # GEMM + in-place all-reduce as two launches
                o = op(a, b, mode="split")
                ctx.check_status()
                report(f"gemm_ar/M{M}/split/{it}", close(o, part))
            keep = op(a, b).clone()         # "auto": whichever the world size selects
            ctx.check_status()
            report(f"gemm_ar/M{M}/auto", close(keep, part))

    @guarded("moe")
    def t_moe():
        from commbench_b200.ops.moe import MoELayer, reference_moe, router_topk

        T, H, I, E, K = 256, 1024, 512, 8 * world, 4
        layer = MoELayer(ctx, T, H, I, E, K, capacity_factor=4.0, seed=3)
        g = torch.Generator(device="cuda").manual_seed(500 + rank)
        x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
        idx, w = router_topk(torch.randn(T, E, device="cuda", generator=g), K)
        w1, w2 = layer.weights()
        w1_all = torch.cat(gather_all(w1.contiguous()))
        w2_all = torch.cat(gather_all(w2.contiguous()))
        ref = reference_moe(x, idx, w, w1_all, w2_all, I)
        for it in range(3):
            y = layer.forward(x, idx, w)
            ctx.check_status()
            err = ((y.float() - ref).abs().max() / (ref.abs().max() + 1e-6)).item()
            report(f"moe/{it}", err < 3e-2, err)
        # routed block with a logical -> physical expert map: skew the load, rebalance, and the
        # output for the same tokens must not change (experts moved, the function did not)
        from commbench_b200.parallel.ep import ExpertParallelMoE

        blk = ExpertParallelMoE(ctx, T, H, I, E, K, capacity_factor=4.0, seed=4)
        logits = torch.randn(T, E, device="cuda", generator=g)
        logits[:, :E // world] += 1.0                    # rank 0's experts are hot
        y0 = blk(x, router_logits=logits).clone()
        ctx.check_status()
        info = blk.rebalance()
        y1 = blk(x, router_logits=logits).clone()
        ctx.check_status()
        err = ((y1.float() - y0.float()).abs().max() / (y0.float().abs().max() + 1e-6)).item()
        report("ep/rebalance_keeps_output", err < 1e-2 and info["moved"] > 0 and
               info["imbalance_after"] < info["imbalance_before"], [err, info])

    @guarded("moe_per_token")
    def t_moe_per_token():
        # a token crosses NVLink once per destination rank; the receive kernel expands it
        from commbench_b200.ops.moe import MoELayer, reference_moe, router_topk

        T, H, I, E, K = 256, 1024, 512, 8 * world, 4
        layer = MoELayer(ctx, T, H, I, E, K, capacity_factor=4.0, seed=3, dispatch="per_token")
        g = torch.Generator(device="cuda").manual_seed(500 + rank)
        x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
        idx, w = router_topk(torch.randn(T, E, device="cuda", generator=g), K)
        w1, w2 = layer.weights()
        w1_all = torch.cat(gather_all(w1.contiguous()))
        w2_all = torch.cat(gather_all(w2.contiguous()))
        ref = reference_moe(x, idx, w, w1_all, w2_all, I)
        for it in range(3):
            y = layer.forward(x, idx, w)
            ctx.check_status()
            err = ((y.float() - ref).abs().max() / (ref.abs().max() + 1e-6)).item()
            report(f"moe_per_token/{it}", err < 3e-2, err)

    @guarded("attention")
    def t_attention():
        from commbench_b200.ops.cp import (RingAttention, reference_attention, ulysses_attention,
                                           zigzag_chunks)

        B, Sl, Hq, Hkv = 1, 512, 2 * world, world
        S = Sl * world
        g = torch.Generator(device="cuda").manual_seed(4242)      # same global tensors everywhere
        qg = torch.randn(B, S, Hq, 128, device="cuda", generator=g).bfloat16()
        kg = torch.randn(B, S, Hkv, 128, device="cuda", generator=g).bfloat16()
        vg = torch.randn(B, S, Hkv, 128, device="cuda", generator=g).bfloat16()
        ref, _ = reference_attention(qg, kg, vg, causal=True)
        # contiguous sharding (Ulysses, ring without zigzag)
        sl = slice(rank * Sl, (rank + 1) * Sl)
        q, k, v = qg[:, sl].contiguous(), kg[:, sl].contiguous(), vg[:, sl].contiguous()
        for it in range(3):
            o = ulysses_attention(ctx, q, k, v, causal=True)
            ctx.check_status()
            report(f"ulysses/{it}", torch.allclose(o.float(), ref[:, sl], atol=3e-2, rtol=3e-2),
                   (o.float() - ref[:, sl]).abs().max().item())
        ring = RingAttention(ctx, B, Sl, Hq, Hkv, zigzag=False)
        for it in range(2):
            o, _ = ring.forward(q, k, v, causal=True)
            ctx.check_status()
            report(f"ring/contiguous/{it}", torch.allclose(o.float(), ref[:, sl], atol=3e-2, rtol=3e-2),
                   (o.float() - ref[:, sl]).abs().max().item())
        # zigzag sharding: rank r owns chunks r and 2W-1-r of the sequence
        h = Sl // 2
        a, b = zigzag_chunks(world, rank)
        pick = torch.cat([torch.arange(a * h, (a + 1) * h), torch.arange(b * h, (b + 1) * h)]).cuda()
        qz, kz, vz = (t.index_select(1, pick).contiguous() for t in (qg, kg, vg))
        ringz = RingAttention(ctx, B, Sl, Hq, Hkv, zigzag=True)
        rz = ref.index_select(1, pick)
        for it in range(3):
            o, _ = ringz.forward(qz, kz, vz, causal=True)
            ctx.check_status()
            report(f"ring/zigzag/{it}", torch.allclose(o.float(), rz, atol=3e-2, rtol=3e-2),
                   (o.float() - rz).abs().max().item())
        # the same object without the mask: the plan (pieces to pull) changes
        full, _ = reference_attention(qg, kg, vg, causal=False)
        o, _ = ringz.forward(qz, kz, vz, causal=False)
        ctx.check_status()
        fz = full.index_select(1, pick)
        report("ring/zigzag/full", torch.allclose(o.float(), fz, atol=3e-2, rtol=3e-2),
               (o.float() - fz).abs().max().item())

    @guarded("p2p_probes")
    def t_p2p():
        from commbench_b200.ops import util as U

        us = U.pingpong_latency(ctx, 500)
        report("pingpong", rank >= 2 or (us is not None and 0.5 < us < 200.0), us)
        us2 = U.pingpong_latency(ctx, 500)          # second call continues from the running value
        report("pingpong/again", rank >= 2 or (us2 is not None and 0.5 < us2 < 200.0), us2)
        for mode in ("kernel", "engine"):
            gbs = U.peer_copy_bandwidth(ctx, 64 << 20, mode)
            report(f"peer_copy/{mode}", gbs > 50.0, gbs)
        b = U.barrier_latency(ctx, 200, False)
        report("barrier_latency", 0.5 < b < 500.0, b)
        if ctx.has_multicast:
            b = U.barrier_latency(ctx, 200, True)
            report("barrier_latency/nvls", 0.5 < b < 500.0, b)

    @guarded("parallel")
    def t_parallel():
        from commbench_b200.parallel import dp, tp

        # ---- data parallel: gradients accumulate straight into symmetric buckets
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.ReLU(),
                                    torch.nn.Linear(512, 64)).cuda()
        buckets = dp.GradBuckets(ctx, model.parameters(), bucket_bytes=256 << 10)
        g = torch.Generator(device="cuda").manual_seed(900 + rank)
        x = torch.randn(32, 256, device="cuda", generator=g)
        model(x).square().mean().backward()
        ref = [p.grad.detach().clone() for p in model.parameters()]
        for r in ref:
            dist.all_reduce(r)
        shards = None
        if all(b.numel() % world == 0 for b in buckets.buckets):
            keep = [b.clone() for b in buckets.buckets]
            shards = buckets.reduce_scatter(average=False)
            for b, k in zip(buckets.buckets, keep):
                b.copy_(k)
        buckets.all_reduce(average=False)
        ctx.check_status()
        ok = all(torch.allclose(p.grad, r, rtol=1e-4, atol=1e-5) for p, r in zip(model.parameters(), ref))
        report("dp/grad_all_reduce", ok and len(buckets.buckets) >= 2, len(buckets.buckets))
        if shards is not None:
            ok = True
            for i, sh in enumerate(shards):
                lo, hi = buckets.shard_range(i)
                ok = ok and torch.allclose(sh, buckets.buckets[i][lo:hi], rtol=1e-4, atol=1e-5)
            report("dp/grad_reduce_scatter", ok)
        lin = torch.nn.Linear(128, 128, bias=False).cuda().bfloat16()
        sp = dp.ShardedParams(ctx, lin.parameters())
        sp.flat.zero_()
        sp.local_shard().fill_(rank + 1)
        sp.all_gather()
        ctx.check_status()
        n = sp.total // world
        want = torch.arange(1, world + 1, device="cuda").repeat_interleave(n).to(sp.flat.dtype)
        report("dp/param_all_gather", torch.equal(sp.flat, want) and lin.weight.data_ptr() == sp.flat.data_ptr())
        # ---- tensor parallel linear layers
        T, H, F = 128 * world, 512, 1024
        col = tp.ColumnParallelLinear(ctx, H, F, T, seed=5)
        row = tp.RowParallelLinear(ctx, F, H, T, scatter_rows=True, seed=6)
        rep = tp.RowParallelLinear(ctx, F, H, T, scatter_rows=False, seed=6)
        xl = rnd((T // world, H), 700 + rank, 1.0)
        xg = torch.cat(gather_all(xl))
        h = col(xl)
        ctx.check_status()
        report("tp/column", close(h, xg.float() @ col.weight.float().t()))
        y = row(h)
        yr = rep(h)
        ctx.check_status()
        full = h.float() @ row.weight.float().t()
        dist.all_reduce(full)
        report("tp/row_scatter", close(y, full[rank * (T // world):(rank + 1) * (T // world)]))
        report("tp/row_replicated", close(yr, full))
        # ---- flagship block end to end: pinned host tokens in, metric out; the chunk-pipelined
        # schedule must give the metric of the single-shot forward, fused and unfused
        from commbench_b200.models.tp_mlp import TPMLP

        Tm = 4096 * world if world <= 4 else 1024 * world
        mlp = TPMLP(ctx, hidden=1024, intermediate=512 * world, max_tokens=Tm, seed=9)
        xh = (torch.randn(Tm // world, 1024, generator=torch.Generator().manual_seed(40 + rank)) * 0.5
              ).bfloat16().pin_memory()
        want = mlp.forward(xh.cuda()).float().abs().mean().item()
        got_f = mlp.forward_host(xh, fused=True)
        got_u = mlp.forward_host(xh, fused=False)
        ctx.check_status()
        report("tp_mlp/forward_host", abs(got_f - want) <= 2e-3 * abs(want) and
               abs(got_u - want) <= 2e-2 * abs(want), [mlp.host_chunks(Tm // world), want, got_f, got_u])
        mlp.gate_host_copy = True      # AG->GEMM launched while the tokens are still on the wire
        got_g = [mlp.forward_host(xh, fused=True) for _ in range(3)]
        ctx.check_status()
        report("tp_mlp/forward_host_gated", all(abs(g - want) <= 2e-3 * abs(want) for g in got_g), got_g)

    groups = {"moe": t_moe, "attention": t_attention, "p2p": t_p2p, "parallel": t_parallel,
              "all_reduce": t_all_reduce, "all_gather": t_all_gather,
              "reduce_scatter": t_reduce_scatter, "all_to_all": t_all_to_all,
              "broadcast": t_broadcast, "ag_gemm": t_ag_gemm, "gemm_rs": t_gemm_rs,
              "gemm_ar": t_gemm_ar}
    on_request = {"moe_per_token": t_moe_per_token}
    wanted = [a for a in sys.argv[1:] if not a.startswith("-")]
    groups.update({k: v for k, v in on_request.items() if k in wanted})
    unknown = [a for a in wanted if a not in groups]
    if unknown:
        raise SystemExit(f"unknown group(s) {unknown}; choose from {sorted(groups)}")
    for name, fn in groups.items():
        if not wanted or name in wanted:
            fn()
    torch.cuda.synchronize()
    dist.barrier()
    ctx.close()
    ok = all(RESULTS)
    if rank == 0:
        print(json.dumps({"summary": "PASS" if ok else "FAIL", "checks": len(RESULTS)}), flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok else 2)


if __name__ == "__main__":
    main()
