"""Tensor-parallel QK RMS-norm in one kernel: every rank holds a slice of the query and key
channels of each token, the norm needs the sum of squares over ALL ranks' channels, so each
CTA pushes its two partial sums (8 bytes) to every peer, waits (bounded) for theirs and
normalises its slice in place.  Here with W virtual ranks inside one cooperative launch on ONE
GPU.  Prints one JSON object.

Reference counterpart: datasets/example101_sglang_qknorm_fused_easy (``parallel_qknorm_across_head``,
8-byte push all-reduce at :147-161, kernel at :205) and datasets/example102_sglang_qknorm_fused_hard.

Run as: python ref_tp_qknorm_virtual_ranks.py
"""
import json

import torch

WORLD = 4
Q_LOCAL, K_LOCAL = 6144 // 8, 1024 // 8
TOKENS = (16, 64, 128)          # W * tokens CTAs must be resident together (one cooperative launch)


class FusedQkNorm:
    def __init__(self):
        from commbench_b200.ops.fused import TPQKNorm
        from commbench_b200.runtime.context import EmuContext

        # --- solution: an EmuContext of WORLD virtual ranks and TPQKNorm for up to max(TOKENS) tokens
        self.ctx = EmuContext(WORLD)
        self.op = TPQKNorm(self.ctx, max_tokens=max(TOKENS), q_local=Q_LOCAL, k_local=K_LOCAL, eps=1e-6)
        # --- end solution

    def run(self, q: list, k: list, wq: list, wk: list):
        """Normalises q[r] [T, Q_LOCAL] and k[r] [T, K_LOCAL] IN PLACE for every virtual rank r."""
        # --- solution: one call for all ranks, then check the device status word
        self.op(q, k, wq, wk)
        self.ctx.check_status()
        # --- end solution


def main():
    if not torch.cuda.is_available():
        print(json.dumps({"Correctness": "SKIP", "reason": "no CUDA device", "metrics": []}))
        return
    from commbench_b200.ops.fused import reference_qknorm

    fused = FusedQkNorm()
    ok, rows = True, []
    for call, T in enumerate(TOKENS):
        g = torch.Generator(device="cuda").manual_seed(call)
        mk = lambda n: [torch.randn(T, n, device="cuda", generator=g).bfloat16() for _ in range(WORLD)]
        q, k = mk(Q_LOCAL), mk(K_LOCAL)
        wq = [torch.rand(Q_LOCAL, device="cuda", generator=g).add(0.5).bfloat16() for _ in range(WORLD)]
        wk = [torch.rand(K_LOCAL, device="cuda", generator=g).add(0.5).bfloat16() for _ in range(WORLD)]
        rq, rk = reference_qknorm(q, k, wq, wk, 1e-6)
        fused.run(q, k, wq, wk)
        torch.cuda.synchronize()
        for r in range(WORLD):
            ok &= torch.allclose(q[r].float(), rq[r], atol=3e-2, rtol=3e-2)
            ok &= torch.allclose(k[r].float(), rk[r], atol=3e-2, rtol=3e-2)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fused.run(q, k, wq, wk)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 100.0
        nbytes = WORLD * T * (Q_LOCAL + K_LOCAL) * 2 * 2
        rows.append({"data_size": T, "latency_avg": us, "throughput_avg": nbytes / (us * 1e-6) / 1e9})
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "tokens", "latency_unit": "us",
                      "throughput_unit": "GB/s", "metrics": rows}))


if __name__ == "__main__":
    main()
