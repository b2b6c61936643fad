"""Pipeline parallelism: hand-off of activations between stages.

Point-to-point traffic stays on NCCL (send / recv on a side stream so it overlaps compute);
tensor dictionaries travel as metadata on the CPU group plus one NCCL message per tensor, the
scheme of the reference's pipeline example
(datasets/example085_vllm_pp_send_recv_tensor_dict/empty_vllm_pp_send_recv_tensor_dict.py:1-36).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops.p2p import recv, recv_tensor_dict, send, send_tensor_dict  # noqa: F401


class PipelineStage:
    """One stage of a linear pipeline over the ranks of ``group`` (stage i = rank i)."""

    def __init__(self, group=None, cpu_group=None):
        self.group, self.cpu_group = group, cpu_group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

    @property
    def is_first(self) -> bool:
        return self.rank == 0

    @property
    def is_last(self) -> bool:
        return self.rank == self.world - 1

    def recv_from_prev(self, device=None) -> dict | None:
        if self.is_first:
            return None
        return recv_tensor_dict(self.rank - 1, device=device, group=self.group, cpu_group=self.cpu_group)

    def send_to_next(self, tensors: dict):
        if not self.is_last:
            send_tensor_dict(tensors, self.rank + 1, group=self.group, cpu_group=self.cpu_group)

    def run(self, fn, first_input: dict | None = None, device=None) -> dict | None:
        """Receives from the previous stage (or takes ``first_input``), applies ``fn`` and sends
        the result on; the last stage returns it."""
        x = first_input if self.is_first else self.recv_from_prev(device)
        y = fn(x)
        if self.is_last:
            return y
        self.send_to_next(y)
        return None
