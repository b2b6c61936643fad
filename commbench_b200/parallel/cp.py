"""Context parallelism for attention over a sequence sharded across ranks: ring (K/V chunks
pulled from their owners while the previous chunk is attended to, exact log-sum-exp merge,
optional zig-zag causal balancing) and Ulysses (sequence <-> head all-to-all around a local
full-sequence attention).

Reference counterparts (communication halves only):
datasets/example057_thunderkitten_ring_attn_easy, datasets/example058_thunderkitten_ulysses_attn_easy.
"""
from ..ops.cp import (RingAttention, attn_merge, flash_attention, reference_attention,  # noqa: F401
                      ulysses_attention, zigzag_chunks)


class ContextParallelAttention:
    """``mode`` = "ring" or "ulysses"; tensors are ``[B, S / W, H, 128]`` bf16."""

    def __init__(self, ctx, batch: int, s_local: int, hq: int, hkv: int, mode: str = "ulysses",
                 zigzag: bool = False):
        if mode not in ("ring", "ulysses"):
            raise ValueError("mode must be 'ring' or 'ulysses'")
        self.ctx, self.mode = ctx, mode
        self._ring = RingAttention(ctx, batch, s_local, hq, hkv, zigzag=zigzag) if mode == "ring" else None

    def __call__(self, q, k, v, causal: bool = True):
        if self._ring is not None:
            return self._ring.forward(q, k, v, causal=causal)[0]
        return ulysses_attention(self.ctx, q, k, v, causal=causal)
