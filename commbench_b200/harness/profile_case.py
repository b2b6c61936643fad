"""One small, self-contained launch sequence per hot kernel, for profiler captures.

    python -m commbench_b200.harness.profile_case gemm   [--m 8192 --n 8192 --k 4096]
    python -m commbench_b200.harness.profile_case gemm_fp8
    python -m commbench_b200.harness.profile_case attn   [--seq 8192 --heads 16]
    python -m commbench_b200.harness.profile_case quant
    python -m commbench_b200.harness.profile_case moe    [--tokens 4096] [--dispatch both]   # per-stage event times
    python -m commbench_b200.harness.profile_case ag_gemm | gemm_rs | gemm_ar  [--world 2]
                                  # the fused kernels, virtual ranks inside ONE cooperative launch

Each case allocates inputs larger than the 126 MB L2 but well under a few GB, runs two warm-up
launches and ``--launches`` measured ones (default 3), prints the CUDA-event time and exits.
Single GPU, single process, no kernel that waits on another rank: safe to run under a
multi-pass profiler (``ncu --set full --clock-control none -k regex:<kernel> -c 3 ...``) once
the plain run has exited 0.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def _time(fn, launches: int) -> float:
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / launches


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "gemm_fp8", "attn", "quant", "moe", "ag_gemm",
                                     "gemm_rs", "gemm_ar"])
    ap.add_argument("--world", type=int, default=2, help="virtual ranks of the fused cases")
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--dispatch", choices=["per_pair", "per_token", "both"], default="per_pair",
                    help="moe: dispatch form(s) to time (per_token = one row per token and rank)")
    ap.add_argument("--bn", type=int, default=0,
                    help="gemm tile selector (0 = chosen from the shape; 512 = CTA pair, 256x256); "
                         "the fused cases take it too (256 = one CTA per 128x256 tile: the form "
                         "a profiler can replay, a cooperative launch without clusters)")
    a = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    out: dict = {"case": a.case}

    if a.case in ("gemm", "gemm_fp8"):
        from ..ops.gemm import gemm

        A = torch.randn(a.m, a.k, device=dev, generator=g)
        B = torch.randn(a.n, a.k, device=dev, generator=g) * 0.05
        if a.case == "gemm_fp8":
            A, B = A.to(torch.float8_e4m3fn), B.to(torch.float8_e4m3fn)
        else:
            A, B = A.bfloat16(), B.bfloat16()
        C = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=dev)
        ms = _time(lambda: gemm(A, B, out=C, bn=a.bn), a.launches)
        out.update(shape=[a.m, a.n, a.k], bn=a.bn, ms=ms, tflops=2.0 * a.m * a.n * a.k / ms / 1e9)
    elif a.case == "attn":
        from ..ops.cp import flash_attention

        q = torch.randn(1, a.seq, a.heads, 128, device=dev, generator=g).bfloat16()
        k = torch.randn(1, a.seq, a.heads // 4, 128, device=dev, generator=g).bfloat16()
        v = torch.randn(1, a.seq, a.heads // 4, 128, device=dev, generator=g).bfloat16()
        ms = _time(lambda: flash_attention(q, k, v, causal=True), a.launches)
        out.update(shape=[1, a.seq, a.heads, a.heads // 4, 128], ms=ms,
                   tflops=4.0 * a.seq * a.seq * 128 * a.heads / 2 / ms / 1e9)
    elif a.case in ("ag_gemm", "gemm_rs", "gemm_ar"):
        # W virtual ranks on this one GPU share its SMs, so the rate to compare with is the
        # plain GEMM's on 148 / W SMs; what the capture shows is the kernel's own behaviour
        # (tensor pipe, DRAM bytes against the algorithmic bytes, stalls on flags).
        from ..ops.tp import AgGemm, GemmAr, GemmRs
        from ..runtime.context import EmuContext

        W = a.world
        ctx = EmuContext(W)
        m, n, k = a.m // 2, a.n // 2, a.k          # 4096 x 4096 x 4096 by default
        if a.case == "ag_gemm":
            op = AgGemm(ctx, max_m=m, k=k)
            A = [torch.randn(m // W, k, device=dev, generator=g).bfloat16() for _ in range(W)]
            B = [(torch.randn(n, k, device=dev, generator=g) * 0.05).bfloat16() for _ in range(W)]
            flops = 2.0 * W * m * n * k
        else:
            op = (GemmRs if a.case == "gemm_rs" else GemmAr)(ctx, m, n)
            A = [torch.randn(m, k // W, device=dev, generator=g).bfloat16() for _ in range(W)]
            B = [(torch.randn(n, k // W, device=dev, generator=g) * 0.05).bfloat16() for _ in range(W)]
            flops = 2.0 * m * n * k
        kw = {"bn": a.bn} if a.bn else {}
        ms = _time(lambda: op(A, B, **kw), a.launches)
        ctx.check_status()
        out.update(world=W, shape=[m, n, k], bn=a.bn, ms=ms, tflops_all_ranks=flops / ms / 1e9)
    elif a.case == "quant":
        from ..ops.gemm import dequantize_blockscaled, quantize_blockscaled

        x = torch.randn(32768, 7168, device=dev, generator=g).bfloat16()
        qx, s = quantize_blockscaled(x, 1)
        y = torch.empty_like(x)
        ms_q = _time(lambda: quantize_blockscaled(x, 1), a.launches)
        ms_d = _time(lambda: dequantize_blockscaled(qx, s, 1, out=y), a.launches)
        nbytes = x.numel() * 3
        out.update(rows=32768, cols=7168, quant_ms=ms_q, dequant_ms=ms_d,
                   quant_gbs=nbytes / ms_q / 1e6, dequant_gbs=nbytes / ms_d / 1e6)
    elif a.case == "moe":
        # One rank's share of the 256-expert layer on one GPU (all traffic local): 4096 tokens,
        # top-8 over the rank's 32 experts = 32,768 expert rows, with per-stage CUDA events.
        from ..ops.moe import MoELayer, router_topk
        from ..runtime.context import EmuContext

        T, H, I, E, K = a.tokens, 7168, 2048, 32, 8
        runs = []
        if a.dispatch in ("per_pair", "both"):
            runs += [("separate_swiglu", False, "per_pair"), ("fused_swiglu", True, "per_pair")]
        if a.dispatch in ("per_token", "both"):
            runs += [("fused_swiglu_per_token", True, "per_token")]
        for label, fused, dispatch in runs:
            ctx = EmuContext(1)
            layer = MoELayer(ctx, T, H, I, E, K, capacity_factor=1.5, fused_swiglu=fused,
                             dispatch=dispatch)
            gg = torch.Generator(device=dev).manual_seed(7)
            x = torch.randn(T, H, device=dev, generator=gg).bfloat16()
            idx, w = router_topk(torch.randn(T, E, device=dev, generator=gg), K)
            for _ in range(3):
                layer.forward([x], [idx], [w])
            torch.cuda.synchronize()
            layer.enable_stage_timing()
            ms = _time(lambda: layer.forward([x], [idx], [w]), a.launches)
            n = a.launches + 2
            stages = {k: round(v / n, 3) for k, v in layer.stage_ms().items()}
            ctx.check_status()
            out[label] = {"ms": round(ms, 3), "stages_ms": stages,
                          "launches_per_call": layer.launches_per_call}
            del layer, ctx
            torch.cuda.empty_cache()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
