"""Fused tensor-parallel GEMMs on fp8 (e4m3) operands with block scales: 1x128 scales on the
activations, 128x128 scales on the weights (the DeepSeek-V3 recipe the target configurations
name).

Operands are STORED as fp8 + fp32 scales (half the bytes in HBM and in checkpoints) and expanded
to bf16 by a bandwidth-bound kernel right before the fused bf16 tcgen05 kernel; a static weight is
expanded once and cached.  The activation expansion reads N bytes and writes 2N (for the
8192 x 8192 activation of the target shape: 64 MB in, 128 MB out, ~30 us at HBM speed, against
~400 us for the fused GEMM).  A mainloop that feeds fp8 tiles and applies the scales per K block
inside the kernel is the next step; the per-tensor-scale fp8 mainloop (``kind::f8f6f4``) already
exists and is reachable through the same ops by passing fp8 tensors directly.

The reference's fp8 fused examples use per-tensor fp8 only
(datasets/example052_thunderkitten_ag_gemm_fp8_easy, example055_thunderkitten_gemm_rs_fp8_easy).
"""
from __future__ import annotations

import torch

from .gemm import dequantize_blockscaled, quantize_blockscaled  # noqa: F401


class BlockScaledWeight:
    """An fp8 weight [N, K] with 128x128 scales and its cached bf16 expansion."""

    def __init__(self, q: torch.Tensor, s: torch.Tensor):
        self.q, self.s = q, s
        self._bf16: torch.Tensor | None = None

    @classmethod
    def from_bf16(cls, w: torch.Tensor) -> "BlockScaledWeight":
        q, s = quantize_blockscaled(w, 128)
        return cls(q, s)

    def bf16(self) -> torch.Tensor:
        if self._bf16 is None:
            self._bf16 = dequantize_blockscaled(self.q, self.s, 128)
        return self._bf16

    def drop_cache(self):
        self._bf16 = None


def _expand_act(a_q, a_s):
    if isinstance(a_q, (list, tuple)):               # rank emulation: one tensor per virtual rank
        return [dequantize_blockscaled(q, s, 1) for q, s in zip(a_q, a_s)]
    return dequantize_blockscaled(a_q, a_s, 1)


def fused_blockscaled(op, a_q, a_s, weight, **kw):
    """Runs a fused GEMM+collective op (``AgGemm``, ``GemmRs`` or ``GemmAr`` instance) on an
    fp8 activation with 1x128 scales and a ``BlockScaledWeight`` (or a list of them under rank
    emulation).  Returns what the op returns."""
    a = _expand_act(a_q, a_s)
    b = [w.bf16() for w in weight] if isinstance(weight, (list, tuple)) else weight.bf16()
    return op(a, b, **kw)
