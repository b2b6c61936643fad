"""Correctness + performance harness: runs a suite of ops on seeded random inputs, checks each
against an fp32/fp64 or NCCL reference, times ours and the unfused NCCL(+cuBLAS) baseline on the
device (CUDA events, max over ranks, warm-up first), and writes ``summary.json`` / ``summary.csv``
with speed-up, bytes/FLOPs, fraction of roofline and verdict per entry.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        -m commbench_b200.harness.run --suite allreduce,coll,p2p,tp,moe,cp --out results/w8

Suites follow the five target configurations (all-reduce sweep; tensor-parallel fused GEMMs;
MoE layer; context-parallel attention) plus ``coll`` for the other collectives and ``p2p`` for
the ping-pong / peer-copy / barrier probes.  One process per GPU; with W=1 the multi-rank
entries degenerate to their local kernels.

Replaces the reference's per-example ``build_and_run.py --compare`` loop (ref vs generated
rebuilt and rerun back to back: datasets/example001_gpu_comm_single_process/nv/build_and_run.py:488-693)
with "ours vs baseline" in one process.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--suite", default="allreduce,tp")
    ap.add_argument("--out", default="results/harness")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--quick", action="store_true", help="coarser sweeps (every 4th size)")
    ap.add_argument("--graphs", action="store_true",
                    help="also time small all-reduces replayed from CUDA graphs (ours and NCCL)")
    ap.add_argument("--scale", type=float, default=1.0,
                    help="shrink the MoE / attention shapes (1.0 = the target configurations)")
    ap.add_argument("--resume", action="store_true",
                    help="skip the suites that every rank finished in an earlier run into --out")
    args = ap.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from ..baseline import nccl as base
    from ..ops import collectives as coll
    from ..runtime.context import CommContext
    from . import report, roofline

    ctx = CommContext(heap_bytes=4 << 30)
    peaks = roofline.load_peaks()
    store = report.ResultStore(os.path.join(args.out, f"results_rank{rank}.jsonl"))

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn) -> float:
        """Mean device time per call over ``--iters`` calls (CUDA events), maximum over ranks;
        the better of two such batches, so that one stray host hiccup (an allocator trim, a
        watchdog wake-up) inside a batch of microsecond-sized calls does not become the number."""
        for _ in range(args.warmup):
            fn()
        best = None
        for _ in range(2):
            sync_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.iters):
                fn()
            e1.record()
            sync_all()
            ms = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            best = float(ms.item()) if best is None else min(best, float(ms.item()))
        return best

    def all_ok(flag: bool) -> bool:
        t = torch.tensor([1 if flag else 0], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    def gather(x):
        if world == 1:
            return [x]
        outs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(outs, x)
        return outs

    def record(op, variant, shape, dtype, **kw):
        rec = dict(key=report.config_key(op, variant, shape, dtype, world), op=op, variant=variant,
                   shape=list(shape), dtype=dtype, world=world, **kw)
        store.add(rec)
        if rank == 0:
            print(json.dumps({k: (round(v, 5) if isinstance(v, float) else v)
                              for k, v in rec.items() if k != "key"}), flush=True)

    suites = [s.strip() for s in args.suite.split(",") if s.strip()]
    ledger = report.SuiteLedger(store, world, {"quick": args.quick, "graphs": args.graphs,
                                               "scale": args.scale, "iters": args.iters},
                                agree=all_ok, enabled=args.resume)
    todo = [s for s in suites if not ledger.done(s)]
    if rank == 0 and len(todo) != len(suites):
        print(json.dumps({"resumed": True, "skipped": [s for s in suites if s not in todo]}), flush=True)
    all_suites, suites = suites, todo

    # ------------------------------------------------------------- all-reduce sweep
    if "allreduce" in suites:
        step = 2 if args.quick else 1
        sizes = [1 << p for p in range(12, 31, step)]           # 4 KB ... 1 GB
        algos = ["oneshot", "twoshot", "twoshot_push"] + \
            (["nvls"] if ctx.has_multicast else []) + ["auto"]
        if world == 1:
            algos = ["oneshot"]
        sym_full, _ = ctx.empty((sizes[-1] // 2,), torch.bfloat16)
        for nbytes in sizes:
            n = nbytes // 2
            g = torch.Generator(device=dev).manual_seed(rank)
            x = (torch.rand(n, device=dev, generator=g) * 2 - 1).bfloat16()
            ref = None
            if nbytes <= (64 << 20):
                ref = sum(t.float() for t in gather(x))
            sym = sym_full[:n]
            base_ms = timed(lambda: base.all_reduce(x.clone())) if world > 1 else None
            clone_ms = timed(lambda: x.clone()) if world > 1 else 0.0
            if base_ms is not None:
                base_ms = max(base_ms - clone_ms, 1e-6)
            for algo in algos:
                if algo == "oneshot" and nbytes > (16 << 20):
                    continue
                sym.copy_(x)
                sync_all()
                if algo == "oneshot" or (algo == "auto" and coll.plan_all_reduce(
                        ctx, nbytes, True)["algo"] == "oneshot"):
                    out = torch.empty_like(x)
                    y = coll.all_reduce(ctx, sym, out=out, algo=algo)
                    fn = lambda a=algo: coll.all_reduce(ctx, sym, out=out, algo=a)
                else:
                    y = coll.all_reduce(ctx, sym, algo=algo)
                    fn = lambda a=algo: coll.all_reduce(ctx, sym, algo=a)
                ctx.check_status()
                correct, err = True, None
                if ref is not None:
                    err = (y.float() - ref).abs().max().item()
                    correct = all_ok(err <= 2e-2 * max(1.0, ref.abs().max().item()))
                ms = timed(fn)
                ctx.check_status()
                f = roofline.allreduce_bus_factor(world)
                resolved = algo if algo != "auto" else \
                    coll.plan_all_reduce(ctx, nbytes, True)["algo"]
                link = roofline.nvlink_bytes("all_reduce", nbytes, world, nvls=(resolved == "nvls"))
                record("all_reduce", algo, (n,), "bf16", correct=correct, max_err=err, time_ms=ms,
                       baseline_ms=base_ms, busbw_gbs=f * nbytes / (ms * 1e-3) / 1e9,
                       baseline_busbw_gbs=(f * nbytes / (base_ms * 1e-3) / 1e9) if base_ms else None,
                       roofline_frac=roofline.fraction(roofline.roofline_ms(0, link, peaks), ms),
                       roofline_note=f"of {peaks.source}")
                if algo == "auto" and nbytes <= (1 << 20) and world > 1 and args.graphs:
                    # Small messages are launch bound: the same call replayed from a CUDA graph,
                    # against NCCL replayed from a graph as well.
                    from ..utils.graphs import time_graphed

                    gms = time_graphed(fn)
                    gbase = time_graphed(lambda: base.all_reduce(x))
                    ctx.check_status()
                    record("all_reduce", "auto+graph", (n,), "bf16", correct=correct, max_err=err,
                           time_ms=gms, baseline_ms=gbase, busbw_gbs=f * nbytes / (gms * 1e-3) / 1e9,
                           roofline_frac=roofline.fraction(roofline.roofline_ms(0, link, peaks), gms),
                           roofline_note=f"of {peaks.source}")
        ledger.mark("allreduce")

    # ----------------------------------------------------------- other collectives
    if "coll" in suites and world > 1:
        sizes_mb = (16, 256) if args.quick else (1, 16, 64, 256)
        big_rows = (max(sizes_mb) << 20) // (world * 256 * 2) * world
        # Communication buffers live in the symmetric heap (the intended use: no staging copy);
        # "staged" entries take ordinary tensors and pay for the copy into the heap.
        x_sym_full, _ = ctx.empty((big_rows, 256), torch.bfloat16)
        ag_out_full, _ = ctx.empty((big_rows, 256), torch.bfloat16)
        for mb in sizes_mb:
            nbytes = mb << 20
            rows = nbytes // (world * 256 * 2) * world
            x = torch.randn(rows, 256, device=dev).bfloat16()
            shard = x[: rows // world].contiguous()
            x_sym, ag_out = x_sym_full[:rows], ag_out_full[:rows]
            x_sym.copy_(x)
            sync_all()
            forced = ()
            if ctx.has_multicast:
                forced = (
                    ("reduce_scatter", "symmetric-in-nvls", lambda: coll.reduce_scatter(ctx, x_sym, use_nvls=True),
                     lambda: base.reduce_scatter(x), "reduce_scatter", nbytes),
                    ("reduce_scatter", "symmetric-in-plain", lambda: coll.reduce_scatter(ctx, x_sym, use_nvls=False),
                     lambda: base.reduce_scatter(x), "reduce_scatter", nbytes),
                )
            for op, variant, ours, theirs, link_op, size in forced + (
                ("all_gather", "symmetric-out", lambda: coll.all_gather(ctx, shard, out=ag_out),
                 lambda: base.all_gather(shard), "all_gather", nbytes),
                ("all_gather", "staged", lambda: coll.all_gather(ctx, shard),
                 lambda: base.all_gather(shard), "all_gather", nbytes),
                ("reduce_scatter", "symmetric-in", lambda: coll.reduce_scatter(ctx, x_sym),
                 lambda: base.reduce_scatter(x), "reduce_scatter", nbytes),
                ("reduce_scatter", "staged", lambda: coll.reduce_scatter(ctx, x),
                 lambda: base.reduce_scatter(x), "reduce_scatter", nbytes),
                ("all_to_all", "symmetric-in", lambda: coll.all_to_all(ctx, x_sym),
                 lambda: base.all_to_all(x), "all_to_all", nbytes),
                ("all_to_all", "staged", lambda: coll.all_to_all(ctx, x),
                 lambda: base.all_to_all(x), "all_to_all", nbytes),
                ("all_to_all", "symmetric-out", lambda: coll.all_to_all(ctx, x, out=ag_out),
                 lambda: base.all_to_all(x), "all_to_all", nbytes),
            ):
                a, b = ours(), theirs()
                ctx.check_status()
                if op == "reduce_scatter":
                    # fp32 reference: NCCL's bf16 ring rounds after every hop, so two correct bf16
                    # results can differ by several units in the last place.
                    ref32 = base.reduce_scatter(x.float())
                    err = (a.float() - ref32).abs().max().item()
                    correct = all_ok(err <= 2e-2 * max(1.0, ref32.abs().max().item()))
                    del ref32
                else:
                    correct = all_ok(torch.equal(a, b))
                ms, bms = timed(ours), timed(theirs)
                link = roofline.nvlink_bytes(link_op, size, world)
                record(op, variant, tuple(x.shape), "bf16", correct=correct, time_ms=ms,
                       baseline_ms=bms, busbw_gbs=link / (ms * 1e-3) / 1e9,
                       roofline_frac=roofline.fraction(roofline.roofline_ms(0, link, peaks), ms))
        ledger.mark("coll")

    # ------------------------------------------------- point-to-point and barrier probes
    if "p2p" in suites and world > 1:
        from ..ops import util as U

        us = U.pingpong_latency(ctx, 2000)
        t = torch.tensor([us if us is not None else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        record("p2p_pingpong", "peer-store", (1,), "u32", correct=True, time_ms=t.item() / 1e3,
               baseline_ms=None, round_trip_us=t.item())
        for use_nvls in ([False, True] if ctx.has_multicast else [False]):
            b_us = U.barrier_latency(ctx, 1000, use_nvls)
            t = torch.tensor([b_us], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            record("barrier", "nvls" if use_nvls else "flag-matrix", (world,), "u32", correct=True,
                   time_ms=t.item() / 1e3, baseline_ms=None, latency_us=t.item())
        for mb in (1, 256):
            for mode in ("kernel", "engine"):
                gbs = U.peer_copy_bandwidth(ctx, mb << 20, mode)
                t = torch.tensor([gbs], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MIN)
                ms = (mb << 20) / (t.item() * 1e6)
                record("p2p_copy", mode, (mb << 20,), "u8", correct=True, time_ms=ms, baseline_ms=None,
                       busbw_gbs=t.item(),
                       roofline_frac=t.item() / peaks.nvlink_gbs)
        ledger.mark("p2p")

    # ------------------------------------------------- tensor-parallel fused GEMMs
    if "tp" in suites:
        from ..ops.gemm import gemm
        from ..ops.tp import AgGemm, GemmAr, GemmRs

        def rnd(shape, seed, scale=0.02):
            g = torch.Generator(device=dev).manual_seed(seed)
            return (torch.randn(shape, device=dev, generator=g) * scale).bfloat16()

        M, K, N = 8192, 8192, 28672
        a_loc, b1 = rnd((M // world, K), 1 + rank, 1.0), rnd((N // world, K), 100 + rank)
        if world > 1:
            ag = AgGemm(ctx, M, K)
            ours = lambda: ag(a_loc, b1)
            theirs = lambda: base.ag_gemm(a_loc, b1)
        else:
            ours = lambda: gemm(a_loc, b1)
            theirs = lambda: torch.matmul(a_loc, b1.t())
        c, r = ours(), theirs()
        ctx.check_status()
        err = ((c.float() - r.float()).abs().max() / (r.float().abs().max() + 1e-9)).item()
        ms, bms = timed(ours), timed(theirs)
        fl = 2.0 * M * K * (N // world)
        link = roofline.nvlink_bytes("all_gather", M * K * 2, world)
        record("ag_gemm", "bf16", (M, N // world, K), "bf16", correct=all_ok(err < 2e-2), max_err=err,
               time_ms=ms, baseline_ms=bms, tflops=fl / (ms * 1e-3) / 1e12,
               roofline_frac=roofline.fraction(roofline.roofline_ms(fl, link, peaks, True), ms))
        a2, b2 = rnd((M, N // world), 200 + rank, 0.05), rnd((K, N // world), 300 + rank)
        if world > 1:
            rs = GemmRs(ctx, M, K)
            ours = lambda: rs(a2, b2)
            theirs = lambda: base.gemm_rs(a2, b2)
        else:
            ours = lambda: gemm(a2, b2)
            theirs = lambda: torch.matmul(a2, b2.t())
        c, r = ours(), theirs()
        ctx.check_status()
        err = ((c.float() - r.float()).abs().max() / (r.float().abs().max() + 1e-9)).item()
        ms, bms = timed(ours), timed(theirs)
        fl = 2.0 * M * K * (N // world)
        link = roofline.nvlink_bytes("reduce_scatter", M * K * 2, world)
        record("gemm_rs", "bf16", (M, K, N // world), "bf16", correct=all_ok(err < 2e-2), max_err=err,
               time_ms=ms, baseline_ms=bms, tflops=fl / (ms * 1e-3) / 1e12,
               roofline_frac=roofline.fraction(roofline.roofline_ms(fl, link, peaks, True), ms))
        # ---- the same two shapes on fp8 e4m3: one scale per tensor, and 1x128 / 128x128
        # power-of-two block scales applied by the tensor cores.  Baseline: NCCL collective on the
        # fp8 bytes + torch._scaled_mm.  The fp8 roofline takes twice the measured bf16 rate.
        from ..ops.gemm import gemm_fp8_mx, quantize_blockscaled_pow2

        f8 = torch.float8_e4m3fn
        one = torch.ones(1, device=dev)

        def smm(x, w):
            return torch._scaled_mm(x, w.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)

        def bs_ref_rows(q, sfw, rows):
            """fp32 rows `rows` of a block-scaled operand (packed exponent words -> scales)."""
            from ..ops.gemm import sf_exponents
            e = sf_exponents(sfw, q.shape[1] // 128)[rows].float()
            return q[rows].float() * torch.exp2(e - 127.0).repeat_interleave(128, dim=1)

        aq, _, asf = quantize_blockscaled_pow2(a_loc, 1)
        b1q, _, b1sf = quantize_blockscaled_pow2(b1, 128)
        a2q, _, a2sf = quantize_blockscaled_pow2(a2, 1)
        b2q, _, b2sf = quantize_blockscaled_pow2(b2, 128)
        sample = torch.arange(0, M // world, max(1, M // world // 64), device=dev)
        if world > 1:
            ag8 = AgGemm(ctx, M, K, dtype=f8)

            def base_ag8():
                full = torch.empty(M, K, dtype=torch.uint8, device=dev)
                dist.all_gather_into_tensor(full, aq.view(torch.uint8))
                return smm(full.view(f8), b1q)

            def base_rs8():
                part = smm(a2q, b2q)
                y = torch.empty(M // world, K, dtype=torch.bfloat16, device=dev)
                dist.reduce_scatter_tensor(y, part)
                return y
            cases = (
                ("ag_gemm", "fp8-per-tensor", lambda: ag8(aq, b1q), base_ag8, (M, N // world, K),
                 "all_gather", M * K),
                ("ag_gemm", "fp8-blockscaled", lambda: ag8(aq, b1q, a_sf=asf, b_sf=b1sf), base_ag8,
                 (M, N // world, K), "all_gather", M * K),
                ("gemm_rs", "fp8-per-tensor", lambda: rs(a2q, b2q), base_rs8, (M, K, N // world),
                 "reduce_scatter", M * K * 2),
                ("gemm_rs", "fp8-blockscaled", lambda: rs(a2q, b2q, a_sf=a2sf, b_sf=b2sf), base_rs8,
                 (M, K, N // world), "reduce_scatter", M * K * 2),
            )
        else:
            cases = (
                ("ag_gemm", "fp8-per-tensor", lambda: gemm(aq, b1q), lambda: smm(aq, b1q),
                 (M, N, K), "all_gather", 0),
                ("ag_gemm", "fp8-blockscaled", lambda: gemm_fp8_mx(aq, asf, b1q, b1sf),
                 lambda: smm(aq, b1q), (M, N, K), "all_gather", 0),
                ("gemm_rs", "fp8-per-tensor", lambda: gemm(a2q, b2q), lambda: smm(a2q, b2q),
                 (M, K, N), "reduce_scatter", 0),
                ("gemm_rs", "fp8-blockscaled", lambda: gemm_fp8_mx(a2q, a2sf, b2q, b2sf),
                 lambda: smm(a2q, b2q), (M, K, N), "reduce_scatter", 0),
            )
        for op_name, variant, ours, theirs, shape, coll_name, coll_bytes in cases:
            c = ours()
            ctx.check_status()
            if variant == "fp8-per-tensor":
                r = theirs()
                err = ((c.float() - r.float()).abs().max() / (r.float().abs().max() + 1e-9)).item()
            elif op_name == "ag_gemm" and world == 1:
                # sampled rows against the fp32 product of the same quantised, scaled operands
                r = bs_ref_rows(aq, asf, sample) @ bs_ref_rows(b1q, b1sf, slice(None)).t()
                err = ((c[sample].float() - r).abs().max() / (r.abs().max() + 1e-9)).item()
            elif op_name == "gemm_rs" and world == 1:
                r = bs_ref_rows(a2q, a2sf, sample) @ bs_ref_rows(b2q, b2sf, slice(None)).t()
                err = ((c[sample].float() - r).abs().max() / (r.abs().max() + 1e-9)).item()
            elif op_name == "ag_gemm":
                # own rows of the gathered product (the other ranks' rows are covered by the
                # per-tensor case and by the virtual-rank tests)
                rows = sample + rank * (M // world)
                r = bs_ref_rows(aq, asf, sample) @ bs_ref_rows(b1q, b1sf, slice(None)).t()
                err = ((c[rows].float() - r).abs().max() / (r.abs().max() + 1e-9)).item()
            else:
                # reduce-scatter: sum over ranks of the sampled rows' partial products
                rows = sample + rank * (M // world)
                part = bs_ref_rows(a2q, a2sf, slice(None)) @ bs_ref_rows(b2q, b2sf, slice(None)).t()
                ref_full = part.clone()
                dist.all_reduce(ref_full)
                r = ref_full[rows]
                err = ((c[sample].float() - r).abs().max() / (r.abs().max() + 1e-9)).item()
                del part, ref_full
            ms, bms = timed(ours), timed(theirs)
            fl = 2.0 * shape[0] * shape[1] * shape[2]
            link = roofline.nvlink_bytes(coll_name, coll_bytes, world) if world > 1 else 0
            record(op_name, variant, shape, "fp8", correct=all_ok(err < 2e-2), max_err=err,
                   time_ms=ms, baseline_ms=bms, tflops=fl / (ms * 1e-3) / 1e12,
                   roofline_frac=roofline.fraction(roofline.roofline_ms(fl / 2, link, peaks, True), ms),
                   note="fp8 roofline = 2 x measured bf16 rate; baseline NCCL + torch._scaled_mm "
                        "with unit scales")
        Kd, Nd = 8192 // world, 8192
        if world > 1:
            ar = GemmAr(ctx, 1024, Nd)
        for Md in (16, 128, 1024):
            a3, b3 = rnd((Md, Kd), 400 + rank, 1.0), rnd((Nd, Kd), 500 + rank)
            for variant in (("oneshot", True), ("twoshot", False), ("split", "split"),
                            ("auto", None)) if world > 1 else (("local", None),):
                if world > 1 and variant[0] == "split":
                    ours = lambda: ar(a3, b3, mode="split")
                elif world > 1:
                    ours = lambda v=variant[1]: ar(a3, b3, oneshot=v)
                    theirs = lambda: base.gemm_ar(a3, b3)
                else:
                    ours = lambda: gemm(a3, b3)
                    theirs = lambda: torch.matmul(a3, b3.t())
                c, r = ours(), theirs()
                ctx.check_status()
                err = ((c.float() - r.float()).abs().max() / (r.float().abs().max() + 1e-9)).item()
                ms, bms = timed(ours), timed(theirs)
                fl = 2.0 * Md * Kd * Nd
                link = roofline.nvlink_bytes("all_reduce", Md * Nd * 2, world)
                record("gemm_ar", variant[0], (Md, Nd, Kd), "bf16", correct=all_ok(err < 2e-2),
                       max_err=err, time_ms=ms, baseline_ms=bms, tflops=fl / (ms * 1e-3) / 1e12,
                       roofline_frac=roofline.fraction(roofline.roofline_ms(fl, link, peaks), ms))
        ledger.mark("tp")

    # ----------------------------------------------------------------- MoE layer
    if "moe" in suites:
        from ..ops.moe import MoELayer, router_topk

        T = max(256, int(4096 * args.scale) // 128 * 128)
        H, I, E, K = 7168, 2048, 256, 8
        layer = MoELayer(ctx, T, H, I, E, K, capacity_factor=1.5)
        g = torch.Generator(device=dev).manual_seed(7 + rank)
        x = torch.randn(T, H, device=dev, generator=g).bfloat16()
        idx, w = router_topk(torch.randn(T, E, device=dev, generator=g), K)
        w1, w2 = layer.weights()
        y = layer.forward(x, idx, w).clone()
        ctx.check_status()
        if world > 1:
            r = base.moe_layer(x, idx, w, w1, w2, E, I)
            theirs = lambda: base.moe_layer(x, idx, w, w1, w2, E, I)
        else:
            from ..ops.moe import reference_moe

            r = reference_moe(x, idx, w, w1, w2, I).bfloat16()
            theirs = None
        err = ((y.float() - r.float()).abs().max() / (r.float().abs().max() + 1e-9)).item()
        ms = timed(lambda: layer.forward(x, idx, w))
        bms = timed(theirs) if theirs else None
        fl = 2.0 * T * K * H * (3 * I)         # per rank, balanced routing
        link = T * K * (world - 1) / world * (H + H * 2)     # fp8 out, bf16 back
        record("moe_layer", "fp8-dispatch", (T, H, I, E, K), "bf16", correct=all_ok(err < 6e-2),
               max_err=err, time_ms=ms, baseline_ms=bms, tflops=fl / (ms * 1e-3) / 1e12,
               roofline_frac=roofline.fraction(roofline.roofline_ms(fl, link, peaks, True), ms))
        ledger.mark("moe")

    # ------------------------------------------------------- context-parallel attention
    if "cp" in suites:
        from ..ops.cp import RingAttention, UlyssesAttention, reference_attention, zigzag_chunks

        Sl = max(512, int(16384 * args.scale) // 512 * 512)
        B, Hq, Hkv = 1, 32, 8
        g = torch.Generator(device=dev).manual_seed(rank)
        q = torch.randn(B, Sl, Hq, 128, device=dev, generator=g).bfloat16()
        k = torch.randn(B, Sl, Hkv, 128, device=dev, generator=g).bfloat16()
        v = torch.randn(B, Sl, Hkv, 128, device=dev, generator=g).bfloat16()
        S = Sl * world
        fl = 4.0 * Sl * S * 128 * Hq / 2            # causal, per rank on average
        theirs = (lambda: base.ulysses_attention(q, k, v)) if world > 1 else \
            (lambda: torch.nn.functional.scaled_dot_product_attention(
                q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),
                is_causal=True, enable_gqa=True))
        r = theirs()
        if world == 1:
            r = r.permute(0, 2, 1, 3)
        bms = timed(theirs)

        def gathered(t):
            if world == 1:
                return [t]
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t)
            return parts

        kparts, vparts = gathered(k), gathered(v)

        def sampled_error(o_local, pieces, kv_pieces):
            """Max error of a few rows of this rank's output against the fp32 attention over the
            whole sequence.  `pieces` = [(first local row, rows, global position)] of this
            rank's queries, `kv_pieces(r)` = the same for rank r's keys."""
            order = sorted((pos, rr, r0, n) for rr in range(world) for (r0, n, pos) in kv_pieces(rr))
            kf = torch.cat([kparts[rr][:, r0:r0 + n] for (_, rr, r0, n) in order], dim=1)
            vf = torch.cat([vparts[rr][:, r0:r0 + n] for (_, rr, r0, n) in order], dim=1)
            worst = 0.0
            for (r0, n, pos) in pieces:
                for off in (0, n - 32):
                    rows = slice(r0 + off, r0 + off + 32)
                    ref, _ = reference_attention(q[:, rows], kf, vf, causal=True,
                                                 q_offset=pos + off, kv_offset=0)
                    worst = max(worst, (o_local[:, rows].float() - ref).abs().max().item())
            return worst

        contiguous = lambda rr: [(0, Sl, rr * Sl)]
        h = Sl // 2
        zz = lambda rr: [(0, h, zigzag_chunks(world, rr)[0] * h),
                         (h, h, zigzag_chunks(world, rr)[1] * h)]

        # Ulysses: inputs placed in the op's symmetric tensors once; a call is one kernel
        # between two cross-GPU barriers, no stand-alone all-to-all.
        uly = UlyssesAttention(ctx, B, Sl, Hq, Hkv)
        uly.q_buf[0].copy_(q)
        uly.k_buf[0].copy_(k)
        uly.v_buf[0].copy_(v)
        o = uly.forward()
        ctx.check_status()
        err = max((o.float() - r.float()).abs().max().item(), sampled_error(o, contiguous(rank), contiguous))
        ms = timed(lambda: uly.forward())
        link = 4 * (world - 1) / world * q.numel() * 2 * (1 + 2 * Hkv / Hq) / 2 if world > 1 else 0
        record("ulysses_attention", "causal", (B, S, Hq, Hkv, 128), "bf16", correct=all_ok(err < 5e-2),
               max_err=err, time_ms=ms, baseline_ms=bms, tflops=fl / (ms * 1e-3) / 1e12,
               roofline_frac=roofline.fraction(roofline.roofline_ms(fl, link, peaks, True), ms))
        del uly
        link2 = (world - 1) * 2 * k.numel() * 2
        for variant, zig, pieces_of in (("causal-contiguous", False, contiguous),
                                        ("causal-zigzag", True, zz)):
            if zig and world == 1:
                continue
            ring = RingAttention(ctx, B, Sl, Hq, Hkv, zigzag=zig)
            ring.k_local().copy_(k)
            ring.v_local().copy_(v)
            o2, _ = ring.forward(q, ring.k_local(), ring.v_local())
            ctx.check_status()
            err2 = sampled_error(o2, pieces_of(rank), pieces_of)
            if not zig:
                err2 = max(err2, (o2.float() - r.float()).abs().max().item())
            ms2 = timed(lambda: ring.forward(q, ring.k_local(), ring.v_local(), want_lse=False))
            record("ring_attention", variant, (B, S, Hq, Hkv, 128), "bf16",
                   correct=all_ok(err2 < 5e-2), max_err=err2, time_ms=ms2, baseline_ms=bms,
                   tflops=fl / (ms2 * 1e-3) / 1e12,
                   roofline_frac=roofline.fraction(roofline.roofline_ms(fl, link2, peaks, True), ms2),
                   note="rows sampled against fp32 attention over the whole sequence")
            del ring
        ledger.mark("cp")

    sync_all()
    if rank == 0:
        s = report.write_summary(store.records(), args.out,
                                 meta={"world": world, "suites": all_suites, "peaks": peaks.__dict__,
                                       "symmetric_memory": {"mode": ctx.mode,
                                                            "multicast": ctx.has_multicast}})
        print(json.dumps({"summary": os.path.join(args.out, "summary.json"),
                          "entries": len(s["entries"]), "all_correct": s["all_correct"],
                          "geomean_speedup": s["geomean_speedup"], "counts": s["counts"]}), flush=True)
    ctx.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
