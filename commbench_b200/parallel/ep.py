"""Expert parallelism: a routed MoE feed-forward block with experts spread over the ranks,
per-expert load accounting and expert re-balancing.

The data path is :class:`~commbench_b200.ops.moe.MoELayer` (deterministic slots -> count matrix
-> plan -> fp8 dispatch push -> dequantising receive -> grouped tcgen05 GEMMs with SwiGLU ->
combine sent from the second GEMM's epilogue -> weighted reduction with optional bias inputs).
This module adds what a model needs around it:

* the router (replicated ``[E, H]`` weight, top-k softmax weights) in front of the layer;
* a logical -> physical expert map, so that experts can move between ranks without the model
  noticing (token routing is translated to physical slots before the dispatch);
* load statistics (tokens per logical expert, summed over ranks) and
  :meth:`ExpertParallelMoE.rebalance`, which computes a greedy longest-processing-time placement
  from them and moves the expert weights with one batched NCCL p2p exchange.

Reference counterparts: datasets/example042_deepep_dispatch_layout, example047_deepep_intranode_notify_dispatch,
example078 ... example083 (DeepEP dispatch / combine stages and their epilogues),
example056_thunderkitten_moe_dispatch_gemm_easy, example089_vllm_eplb_expert_rebalance
(``rearrange_expert_weights_inplace`` over ``batch_isend_irecv``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops.moe import (MoELayer, dispatch_layout, expert_sort, interleave_gate_up,  # noqa: F401
                       reference_moe, router_topk)
from ..ops.p2p import rearrange_expert_weights_inplace  # noqa: F401
from ..runtime.context import CommError


def balanced_placement(load: list[float], world: int) -> list[int]:
    """``new_map[slot] = logical expert``: experts sorted by load, each given to the rank with
    the least load so far that still has a free slot (longest processing time first).  Slots of
    rank r are ``r * E/W ... (r+1) * E/W - 1``.  Deterministic: ties go to the lower index."""
    E = len(load)
    if E % world:
        raise ValueError("experts must divide by the world size")
    per = E // world
    order = sorted(range(E), key=lambda e: (-float(load[e]), e))
    rank_load = [0.0] * world
    rank_slots: list[list[int]] = [[] for _ in range(world)]
    for e in order:
        r = min((r for r in range(world) if len(rank_slots[r]) < per),
                key=lambda r: (rank_load[r], r))
        rank_slots[r].append(e)
        rank_load[r] += float(load[e])
    return [e for r in range(world) for e in sorted(rank_slots[r])]


def imbalance(load: list[float], placement: list[int], world: int) -> float:
    """Largest rank load over the mean rank load (1.0 = perfectly even) under ``placement``."""
    per = len(placement) // world
    rank_load = [sum(float(load[e]) for e in placement[r * per:(r + 1) * per]) for r in range(world)]
    mean = sum(rank_load) / world
    return max(rank_load) / mean if mean > 0 else 1.0


class ExpertParallelMoE(MoELayer):
    """Routed MoE block: ``y = layer(x)`` with ``x`` [T, H] bf16.

    ``shared`` / ``residual`` (optional [T, H] bf16) are added inside the combine reduction -
    the output of a shared expert, a residual stream - instead of by separate kernels."""

    def __init__(self, ctx, tokens: int, hidden: int, intermediate: int, num_experts: int,
                 topk: int, capacity_factor: float = 2.0, seed: int = 0, router_weight=None,
                 dispatch: str = "per_pair"):
        super().__init__(ctx, tokens, hidden, intermediate, num_experts, topk,
                         capacity_factor=capacity_factor, seed=seed, dispatch=dispatch)
        if self.emu:
            raise CommError("ExpertParallelMoE runs on real ranks; use MoELayer for emulation")
        dev = ctx.device
        if router_weight is None:
            g = torch.Generator(device=dev).manual_seed(seed * 31 + 5)     # same on every rank
            router_weight = (torch.randn(num_experts, hidden, device=dev, generator=g) * 0.02)
        self.router_weight = router_weight.to(device=dev, dtype=torch.bfloat16)
        # slot_of[e] = physical slot of logical expert e; placement[slot] = logical expert
        self.placement = list(range(num_experts))
        self.slot_of = torch.arange(num_experts, device=dev, dtype=torch.int32)
        self.load = torch.zeros(num_experts, device=dev, dtype=torch.float32)
        self.track_load = True

    # ------------------------------------------------------------------ forward
    def route(self, x: torch.Tensor):
        """(logical top-k expert ids [T, K] int32, weights [T, K] fp32) of a token batch."""
        logits = torch.matmul(x, self.router_weight.t()).float()
        return router_topk(logits, self.K)

    def __call__(self, x, router_logits=None, shared=None, residual=None):
        if router_logits is None:
            idx, w = self.route(x)
        else:
            idx, w = router_topk(router_logits, self.K)
        if self.track_load:
            self.load += torch.bincount(idx.reshape(-1).long(), minlength=self.E).float()
        phys = self.slot_of[idx.long()]
        return self.forward(x, phys, w, bias0=shared, bias1=residual)

    # ------------------------------------------------------------------ load and placement
    def expert_load(self, group=None) -> list[float]:
        """Tokens routed to each logical expert since the last reset, summed over the ranks."""
        t = self.load.clone()
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(t, group=group)
        return t.tolist()

    def reset_load(self) -> None:
        self.load.zero_()

    def rebalance(self, load: list[float] | None = None, min_gain: float = 0.02, group=None) -> dict:
        """Moves experts so that the measured load is spread evenly (collective: every rank
        calls it with the same ``load``; by default the all-reduced counters).  Nothing moves
        when the expected gain in the max/mean rank load is below ``min_gain``.  Returns
        ``{"moved", "p2p_ops", "imbalance_before", "imbalance_after"}``."""
        load = self.expert_load(group) if load is None else list(load)
        W = self.W
        before = imbalance(load, self.placement, W)
        new_map = balanced_placement(load, W)
        after = imbalance(load, new_map, W)
        if before - after < min_gain:
            return {"moved": 0, "p2p_ops": 0, "imbalance_before": before, "imbalance_after": before}
        torch.cuda.synchronize(self.ctx.device)           # no forward may still read the weights
        st = self.states[0]
        ops = rearrange_expert_weights_inplace(self.placement, new_map, [st.w1, st.w2], self.El,
                                               group=group)
        if st.w1_gated is not None:
            st.w1_gated = interleave_gate_up(st.w1)       # the gated copy follows its source
        moved = sum(1 for a, b in zip(self.placement, new_map) if a != b)
        self.placement = new_map
        inv = [0] * self.E
        for slot, e in enumerate(new_map):
            inv[e] = slot
        self.slot_of.copy_(torch.tensor(inv, dtype=torch.int32))
        self.reset_load()
        return {"moved": moved, "p2p_ops": ops, "imbalance_before": before,
                "imbalance_after": after}
