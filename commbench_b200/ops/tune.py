"""Measures the launch-shape table of the collectives on the machine at hand.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m commbench_b200.ops.tune --out my_table.json
    CB200_TUNE_TABLE=my_table.json python ...        # use it

For every (op, buffer kind, message size) each candidate (algorithm, grid size, vectors in
flight per thread) is timed on the device with CUDA events after warm-up; the time of a
candidate is the maximum over ranks; the fastest one becomes the table row
(:mod:`commbench_b200.ops.tuning` has the layout).  The winner is checked against NCCL's
result of the same op before it is recorded, and NCCL's time is printed beside it.

The search is small on purpose (a few hundred launches of at most a few milliseconds): the
same role as ``NCCL_ALGO`` / the tuner plug-in for the library baseline
(datasets/example019_torch_distributed_nccl_allreduce/empty_nccl_allreduce.py:35-70).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from . import collectives as coll
from . import tuning


def _grid_candidates(per_cta_bytes_total: int, cap: int = 128) -> list[int]:
    """Grid sizes worth trying for a message whose per-rank share is ``per_cta_bytes_total``
    bytes: no CTA gets less than 8 KB.  Grids stop at 128 CTAs: a collective that fills all
    148 SMs measured bimodal (it leaves no SM to whatever else the stream runs, and its
    waiting CTAs are the most pollers a GPU can have)."""
    most = max(1, min(cap, per_cta_bytes_total // 8192))
    least = min(most, per_cta_bytes_total // (2 << 20))     # nor more than 2 MB
    out = [b for b in (4, 8, 16, 32, 64, 96, 128) if least <= b <= most]
    if not out:
        out = [most]
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", required=True, help="table file to write / update")
    ap.add_argument("--ops", default="all_reduce,all_gather,reduce_scatter,all_to_all")
    ap.add_argument("--sizes-kb", default="64,512,4096,16384,65536,262144",
                    help="message sizes in KB (op's own convention: all_reduce / reduce_scatter / "
                         "all_to_all full message, all_gather gathered output)")
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--unrolls", default="2,4,8")
    ap.add_argument("--cand-log", dest="log", default=None, help="JSON-lines file for every measured candidate")
    args = ap.parse_args(argv)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        print("tune: needs at least 2 ranks", file=sys.stderr)
        return 2
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from ..runtime.context import CommContext

    sizes = sorted(int(s) << 10 for s in args.sizes_kb.split(",") if s)
    unrolls = [int(u) for u in args.unrolls.split(",") if u]
    ops = [o.strip() for o in args.ops.split(",") if o.strip()]
    big = max(sizes)
    ctx = CommContext(heap_bytes=3 * big + (64 << 20))
    os.environ["CB200_TUNE_TABLE"] = "off"      # candidates must not be overridden by a table
    tuning.reload()
    logf = open(args.log, "a") if (args.log and rank == 0) else None

    def sync_all():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    def time_many(fns: list) -> list[float]:
        """Times each callable; one MAX reduction over ranks for the whole list."""
        out = []
        for fn in fns:
            for _ in range(args.warmup):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ctx.check_status()
            out.append(e0.elapsed_time(e1) / args.iters)
        t = torch.tensor(out, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def agree(flag: bool) -> bool:
        t = torch.tensor([1 if flag else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    def pick(op: str, kind: str, nbytes: int, cands: list[tuple[dict, object]], check, nccl_fn,
             bus_factor: float):
        """cands: (row, callable).  Returns the best verified row."""
        sync_all()
        times = time_many([fn for _, fn in cands] + [nccl_fn])
        nccl_ms = times[-1]
        order = sorted(range(len(cands)), key=lambda i: times[i])
        if logf:
            for i in order:
                logf.write(json.dumps({"op": op, "kind": kind, "bytes": nbytes, "world": world,
                                       "row": cands[i][0], "ms": round(times[i], 5),
                                       "nccl_ms": round(nccl_ms, 5)}) + "\n")
            logf.flush()
        for i in order:
            row, fn = cands[i]
            ok = agree(check(fn))
            ctx.check_status()
            if ok:
                if rank == 0:
                    gbs = bus_factor * nbytes / (times[i] * 1e-3) / 1e9
                    ngbs = bus_factor * nbytes / (nccl_ms * 1e-3) / 1e9
                    print(json.dumps({"op": op, "kind": kind, "mb": round(nbytes / 2**20, 3),
                                      "best": row, "ms": round(times[i], 4),
                                      "busbw_gbs": round(gbs, 1), "nccl_ms": round(nccl_ms, 4),
                                      "nccl_busbw_gbs": round(ngbs, 1),
                                      "speedup": round(nccl_ms / times[i], 3)}), flush=True)
                return row
            if rank == 0:
                print(json.dumps({"op": op, "kind": kind, "bytes": nbytes, "rejected": row}),
                      flush=True)
        return None

    table: dict[str, list] = {}
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    src_full = (torch.rand(big // 2, device=dev, generator=g) * 2 - 1).bfloat16()
    sym_a, _ = ctx.empty((big // 2,), torch.bfloat16)
    sym_b, _ = ctx.empty((big // 2,), torch.bfloat16)
    plain_out = torch.empty(big // 2, device=dev, dtype=torch.bfloat16)
    W = world

    # ------------------------------------------------------------------ all_reduce
    if "all_reduce" in ops:
        for kind in ("symmetric", "staged"):
            points = []
            for nbytes in sizes:
                n = nbytes // 2
                x = src_full[:n]
                ref = x.float().clone()
                dist.all_reduce(ref)
                sym = sym_a[:n]
                algos = ["twoshot", "twoshot_push"]
                if ctx.has_multicast:
                    algos.append("nvls")
                if nbytes <= (2 << 20):
                    algos.append("oneshot")
                cands = []
                for algo in algos:
                    share = nbytes if algo == "oneshot" else nbytes // W
                    for blocks in _grid_candidates(share):
                        for u in ([4] if algo == "oneshot" else unrolls):
                            row = {"algo": algo, "blocks": blocks, "unroll": u}
                            if kind == "symmetric" and algo != "oneshot":
                                fn = (lambda a=algo, b=blocks, uu=u:
                                      coll.all_reduce(ctx, sym, algo=a, blocks=b, unroll=uu))
                            elif kind == "symmetric":
                                fn = (lambda a=algo, b=blocks, uu=u:
                                      coll.all_reduce(ctx, sym, out=plain_out[:n], algo=a, blocks=b,
                                                      unroll=uu))
                            else:
                                fn = (lambda a=algo, b=blocks, uu=u:
                                      coll.all_reduce(ctx, x, out=plain_out[:n], algo=a, blocks=b,
                                                      unroll=uu))
                            cands.append((row, fn))

                def check(fn, kind=kind, sym=sym, x=x, n=n, ref=ref):
                    if kind == "symmetric":
                        sym.copy_(x)
                    sync_all()
                    y = fn()
                    torch.cuda.synchronize()
                    tol = 2e-2 * max(1.0, ref.abs().max().item())
                    return (y.float() - ref).abs().max().item() <= tol

                nccl_buf = x.clone()
                best = pick("all_reduce", kind, nbytes, cands, check,
                            lambda: dist.all_reduce(nccl_buf), 2.0 * (W - 1) / W)
                if best:
                    points.append((nbytes, best))
            if points:
                table[f"all_reduce@{kind}"] = tuning.make_rows(points)

    # ------------------------------------------------------------------ all_gather
    if "all_gather" in ops:
        for kind in ("push", "pull"):
            points = []
            for total in sizes:
                shard_bytes = total // W // 16 * 16
                if shard_bytes < 16:
                    continue
                n = shard_bytes // 2
                shard = src_full[:n]
                ref = torch.empty(W * n, device=dev, dtype=torch.bfloat16)
                dist.all_gather_into_tensor(ref, shard)
                out = sym_b[:W * n] if kind == "push" else plain_out[:W * n]
                cands = []
                for blocks in _grid_candidates(shard_bytes):
                    for u in unrolls:
                        for mc in ((True, False) if (kind == "push" and ctx.has_multicast) else (None,)):
                            row = {"blocks": blocks, "unroll": u}
                            if mc is not None:
                                row["multicast"] = mc
                            cands.append((row, (lambda b=blocks, uu=u, m=mc:
                                                _ag(ctx, shard, out, b, uu, m))))

                def check(fn, out=out, ref=ref):
                    out.zero_()
                    sync_all()
                    fn()
                    torch.cuda.synchronize()
                    return torch.equal(out, ref)

                nccl_out = torch.empty_like(ref)
                best = pick("all_gather", kind, shard_bytes, cands, check,
                            lambda: dist.all_gather_into_tensor(nccl_out, shard), float(W - 1))
                if best:
                    points.append((shard_bytes, best))
            if points:
                table[f"all_gather@{kind}"] = tuning.make_rows(points)

    # -------------------------------------------------------------- reduce_scatter
    if "reduce_scatter" in ops:
        for kind in ("symmetric", "staged"):
            points = []
            for nbytes in sizes:
                nbytes = nbytes // (16 * W) * (16 * W)
                n = nbytes // 2
                x = src_full[:n].view(W, -1)
                ref = torch.empty(n // W, device=dev, dtype=torch.float32)
                dist.reduce_scatter_tensor(ref, x.float().flatten())
                xin = sym_a[:n].view(W, -1) if kind == "symmetric" else x
                if kind == "symmetric":
                    xin.copy_(x)
                out = plain_out[:n // W].view(1, -1)
                cands = []
                for blocks in _grid_candidates(nbytes // W):
                    for u in unrolls:
                        for nv in ((True, False) if ctx.has_multicast else (False,)):
                            row = {"blocks": blocks, "unroll": u, "nvls": nv}
                            cands.append((row, (lambda b=blocks, uu=u, v=nv: coll.reduce_scatter(
                                ctx, xin, out=out, use_nvls=v, blocks=b, unroll=uu))))

                def check(fn, out=out, ref=ref):
                    out.zero_()
                    sync_all()
                    fn()
                    torch.cuda.synchronize()
                    tol = 2e-2 * max(1.0, ref.abs().max().item())
                    return (out.flatten().float() - ref).abs().max().item() <= tol

                nccl_out = torch.empty(n // W, device=dev, dtype=torch.bfloat16)
                best = pick("reduce_scatter", kind, nbytes, cands, check,
                            lambda: dist.reduce_scatter_tensor(nccl_out, x.flatten()),
                            (W - 1) / W)
                if best:
                    points.append((nbytes, best))
            if points:
                table[f"reduce_scatter@{kind}"] = tuning.make_rows(points)

    # ------------------------------------------------------------------ all_to_all
    if "all_to_all" in ops:
        for kind in ("out_symmetric", "symmetric", "staged"):
            points = []
            for nbytes in sizes:
                nbytes = nbytes // (16 * W) * (16 * W)
                n = nbytes // 2
                x = src_full[:n].view(W, -1)
                ref = torch.empty_like(x)
                dist.all_to_all_single(ref, x)
                xin = sym_a[:n].view(W, -1) if kind == "symmetric" else x
                if kind == "symmetric":
                    xin.copy_(x)
                out = (sym_b if kind == "out_symmetric" else plain_out)[:n].view(W, -1)
                cands = []
                for blocks in _grid_candidates(nbytes // W):
                    for u in unrolls:
                        for push in (True, False):
                            if kind == "out_symmetric" and not push:
                                continue
                            row = {"blocks": blocks, "unroll": u, "push": push}
                            cands.append((row, (lambda b=blocks, uu=u, p=push: coll.all_to_all(
                                ctx, xin, out=out, blocks=b, unroll=uu, push=p))))

                def check(fn, out=out, ref=ref):
                    out.zero_()
                    sync_all()
                    fn()
                    torch.cuda.synchronize()
                    return torch.equal(out, ref)

                nccl_out = torch.empty_like(x)
                best = pick("all_to_all", kind, nbytes, cands, check,
                            lambda: dist.all_to_all_single(nccl_out, x), (W - 1) / W)
                if best:
                    points.append((nbytes, best))
            if points:
                table[f"all_to_all@{kind}"] = tuning.make_rows(points)

    sync_all()
    if rank == 0:
        tuning.merge_into(args.out, world, table)
        print(json.dumps({"tuned": sorted(table), "world": world, "out": args.out}), flush=True)
    if logf:
        logf.close()
    sync_all()
    ctx.close()
    dist.destroy_process_group()
    return 0


def _ag(ctx, shard, out, blocks, unroll, multicast):
    """all_gather with the multicast choice forced (the public op takes it from the table)."""
    if multicast is None:
        return coll.all_gather(ctx, shard, out=out, blocks=blocks, unroll=unroll)
    return coll.all_gather(ctx, shard, out=out, blocks=blocks, unroll=unroll, multicast=multicast)


if __name__ == "__main__":
    raise SystemExit(main())
