"""Context parallelism for attention over a sequence sharded across ranks.

``ContextParallelAttention`` is the strategy object a model layer holds: it owns the symmetric
buffers, hands out the views a projection should write its K / V (ring) or Q / K / V (Ulysses)
into, shards and un-shards full sequences (zig-zag for causal balance), and runs one fused
kernel per call:

* ``mode="ring"``: K/V shards are pulled in ring order by communication CTAs of the attention
  kernel while the other CTAs attend (``ops.cp.RingAttention``);
* ``mode="ulysses"``: head slices of K/V are pulled, Q tiles are loaded from and O rows stored
  to their owners inside the attention kernel (``ops.cp.UlyssesAttention``).

Reference counterparts (communication halves only):
datasets/example057_thunderkitten_ring_attn_easy, datasets/example058_thunderkitten_ulysses_attn_easy.
"""
from __future__ import annotations

import torch

from ..ops.cp import (RingAttention, UlyssesAttention, attn_merge, flash_attention,  # noqa: F401
                      reference_attention, ulysses_attention, zigzag_chunks, zigzag_shard)


class ContextParallelAttention:
    """Tensors are ``[B, S / W, H, 128]`` bf16.  ``zigzag`` applies to the ring mode."""

    def __init__(self, ctx, batch: int, s_local: int, hq: int, hkv: int, mode: str = "ring",
                 zigzag: bool = True):
        if mode not in ("ring", "ulysses"):
            raise ValueError("mode must be 'ring' or 'ulysses'")
        self.ctx, self.mode, self.world = ctx, mode, ctx.world
        self.s_local = s_local
        self.zigzag = bool(zigzag) and mode == "ring" and ctx.world > 1
        if mode == "ring":
            self.op = RingAttention(ctx, batch, s_local, hq, hkv, zigzag=zigzag)
        else:
            self.op = UlyssesAttention(ctx, batch, s_local, hq, hkv)

    # ------------------------------------------------------------- sharding helpers
    def shard(self, x_full: torch.Tensor, rank: int | None = None) -> torch.Tensor:
        """Rows of a full-sequence tensor ``[B, S, ...]`` that ``rank`` (default: this rank) owns."""
        r = self.ctx.rank if rank is None else rank
        if self.zigzag:
            return zigzag_shard(x_full, self.world, r)
        return x_full[:, r * self.s_local:(r + 1) * self.s_local].contiguous()

    def positions(self, rank: int | None = None) -> torch.Tensor:
        """Global sequence position of every local row (for rotary embeddings and the like)."""
        r = self.ctx.rank if rank is None else rank
        dev = self.ctx.device
        if not self.zigzag:
            return torch.arange(r * self.s_local, (r + 1) * self.s_local, device=dev)
        h = self.s_local // 2
        a, b = zigzag_chunks(self.world, r)
        return torch.cat([torch.arange(a * h, (a + 1) * h, device=dev),
                          torch.arange(b * h, (b + 1) * h, device=dev)])

    # --------------------------------------------------- where projections should write
    def kv_views(self):
        """(k, v) views of symmetric memory to write this rank's keys / values into."""
        if self.mode == "ring":
            return self.op.k_local(), self.op.v_local()
        return self.op.k_buf[0], self.op.v_buf[0]

    def q_view(self):
        """Ulysses only: the symmetric query tensor (ring reads ordinary local queries)."""
        return self.op.q_buf[0] if self.mode == "ulysses" else None

    def __call__(self, q, k, v, causal: bool = True):
        if self.mode == "ring":
            return self.op.forward(q, k, v, causal=causal)[0]
        return self.op.forward(q, k, v, causal=causal)
