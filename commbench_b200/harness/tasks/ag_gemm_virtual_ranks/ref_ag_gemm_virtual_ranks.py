"""The fused all-gather + GEMM kernel on ONE GPU: W virtual ranks run inside a single cooperative
launch (the grid is W groups of resident CTAs, each with its own operands, flags and "peer"
pointers), so the cross-rank protocol - communication CTAs publishing row blocks, tensor-core
CTAs waiting for them - is exercised without two launches ever waiting for each other.
Prints one JSON object.

Same exercise as the reference's datasets/example051_thunderkitten_ag_gemm_easy, posed for a
machine with a single GPU.

Run as: python ref_ag_gemm_virtual_ranks.py
"""
import json

import torch

WORLD = 4
M_LOCAL, N_LOCAL, K = 512, 1024, 2048


class VirtualRankAgGemm:
    def __init__(self):
        from commbench_b200.ops.tp import AgGemm
        from commbench_b200.runtime.context import EmuContext

        # --- solution: an EmuContext of WORLD virtual ranks and the fused op built on it
        self.ctx = EmuContext(WORLD)
        self.op = AgGemm(self.ctx, max_m=M_LOCAL * WORLD, k=K)
        # --- end solution

    def run(self, a_locals: list, b_locals: list) -> list:
        """a_locals[r] [M_LOCAL, K], b_locals[r] [N_LOCAL, K] bf16 ->
        outs[r] [WORLD * M_LOCAL, N_LOCAL] = cat(a_locals) @ b_locals[r]^T, one launch for all."""
        # --- solution: call the op with the per-rank lists, then check the device status word
        outs = self.op(a_locals, b_locals)
        self.ctx.check_status()
        return outs
        # --- end solution


def main():
    if not torch.cuda.is_available():
        print(json.dumps({"Correctness": "SKIP", "reason": "no CUDA device", "metrics": []}))
        return
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3)
    a = [(torch.randn(M_LOCAL, K, device=dev, generator=g) * 0.5).bfloat16() for _ in range(WORLD)]
    b = [(torch.randn(N_LOCAL, K, device=dev, generator=g) * 0.05).bfloat16() for _ in range(WORLD)]
    op = VirtualRankAgGemm()
    outs = op.run(a, b)
    torch.cuda.synchronize()
    full = torch.cat(a).float()
    ok = outs is not None and len(outs) == WORLD
    for r in range(WORLD if ok else 0):
        ref = full @ b[r].float().t()
        ok = ok and bool(((outs[r].float() - ref).abs().max() <= 2e-2 * float(ref.abs().max())).item())
    rows = []
    if ok:
        for _ in range(3):
            op.run(a, b)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            op.run(a, b)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 100.0
        fl = 2.0 * WORLD * (WORLD * M_LOCAL) * N_LOCAL * K
        rows.append({"data_size": WORLD * M_LOCAL * K * 2 / 2**20, "latency_avg": us,
                     "throughput_avg": fl / (us * 1e-6) / 1e12})
    print(json.dumps({"Correctness": "PASS" if ok and rows else "FAIL", "data_size_unit": "MB",
                      "latency_unit": "us", "throughput_unit": "TFLOP/s", "metrics": rows}))


if __name__ == "__main__":
    main()
