"""Fused tensor-parallel GEMMs on fp8 (e4m3) operands with block scales: 1x128 scales on the
activations, 128x128 scales on the weights (the DeepSeek-V3 recipe the target configurations
name).

Two forms:

* **power-of-two scales, applied by the tensor cores** (:func:`quantize_act_mx`,
  :class:`MxWeight`, :func:`fused_mx`): the quantised tensors are the MMA operands
  (``tcgen05.mma.kind::mxf8f6f4.block_scale``), the 8-bit scale exponents ride in tensor memory,
  and in the all-gather -> GEMM kernel the scale words of a row block travel to the peers with
  its rows.  Nothing is expanded; this is the path to use.
* **arbitrary fp32 scales through bf16** (:class:`BlockScaledWeight`, :func:`fused_blockscaled`):
  operands are expanded to bf16 by a bandwidth-bound kernel right before the bf16 kernel (a
  static weight once, cached).  Kept for scales that are not powers of two and as a cross-check.

Tensors with one scale per tensor need neither: pass fp8 tensors to ``AgGemm`` / ``GemmRs`` /
``GemmAr`` and fold the scales into ``alpha``.

The reference's fp8 fused examples use per-tensor fp8 only
(datasets/example052_thunderkitten_ag_gemm_fp8_easy, example055_thunderkitten_gemm_rs_fp8_easy).
"""
from __future__ import annotations

import torch

from .gemm import (dequantize_blockscaled, quantize_blockscaled,  # noqa: F401
                   quantize_blockscaled_pow2)


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


# ------------------------------------------------------------- hardware-applied block scales
def quantize_act_mx(x: torch.Tensor):
    """bf16 activation [rows, K] -> (e4m3, packed 1x128 power-of-two scale words)."""
    q, _, sf = quantize_blockscaled_pow2(x, 1)
    return q, sf


class MxWeight:
    """An fp8 weight [N, K] with power-of-two 128x128 block scales in the packed form the
    block-scaled kernels read (one exponent byte per output column and K block)."""

    def __init__(self, q: torch.Tensor, sf: torch.Tensor):
        self.q, self.sf = q, sf

    @classmethod
    def from_bf16(cls, w: torch.Tensor) -> "MxWeight":
        q, _, sf = quantize_blockscaled_pow2(w, 128)
        return cls(q, sf)


def fused_mx(op, a_q, a_sf, weight, **kw):
    """Runs ``AgGemm`` or ``GemmRs`` on fp8 operands whose block scales the tensor cores apply.
    ``a_q`` / ``a_sf`` from :func:`quantize_act_mx`, ``weight`` an :class:`MxWeight` (lists with
    one entry per virtual rank under rank emulation)."""
    if isinstance(weight, (list, tuple)):
        return op(a_q, [w.q for w in weight], a_sf=a_sf, b_sf=[w.sf for w in weight], **kw)
    return op(a_q, weight.q, a_sf=a_sf, b_sf=weight.sf, **kw)
