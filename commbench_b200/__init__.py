"""commbench_b200: a Blackwell-native (sm_100a) multi-GPU communication and
compute-communication fusion library with a PyTorch-facing API.

Layers (bottom up):
  csrc/prim     device primitives (flags, barriers, mbarrier, TMA, tcgen05, multimem)
  csrc/symm     symmetric memory (VMM + fd exchange + NVSwitch multicast) and the broker
  csrc/coll     collective kernels          -> ops.collectives
  csrc/gemm     tcgen05 GEMM core           -> ops.gemm
  csrc/fused    GEMM+collective kernels     -> ops.tp
  csrc/moe      expert-parallel kernels     -> ops.moe
  csrc/attn     attention kernels           -> ops.cp
  csrc/util     FIFOs, probes, shm queue, transports -> ops.util / utils
  harness       correctness + performance harness (registry, verdicts, roofline, reports)
"""
from .config import Config, get_config, set_config  # noqa: F401

__version__ = "0.1.0"
