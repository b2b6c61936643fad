"""Expert parallelism: the MoE feed-forward layer with experts spread over the ranks
(``ops.moe.MoELayer``: deterministic slots -> count matrix -> plan -> fp8 dispatch push ->
dequantising receive -> grouped tcgen05 GEMMs with SwiGLU -> combine sent from the second GEMM's
epilogue -> weighted reduction), plus expert re-balancing over NCCL p2p.

Reference counterparts: datasets/example042_deepep_dispatch_layout, example047_deepep_intranode_notify_dispatch,
example078 ... example083 (DeepEP dispatch / combine stages), example056_thunderkitten_dispatch_gemm_easy,
example089_vllm_eplb_expert_rebalance.
"""
from ..ops.moe import (MoELayer, dispatch_layout, expert_sort, reference_moe,  # noqa: F401
                       router_topk)
from ..ops.p2p import rearrange_expert_weights_inplace  # noqa: F401


class ExpertParallelMoE(MoELayer):
    """``MoELayer`` that also routes: ``layer(x, router_logits)``."""

    def __call__(self, x, router_logits):
        idx, w = router_topk(router_logits, self.K)
        return self.forward(x, idx, w)
