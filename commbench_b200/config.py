"""Typed configuration with ``CB200_*`` environment overrides.

The reference has no central configuration: every example script parses its own
argparse flags and environment variables (scripts/generate_eval_one.py:661-753,
datasets/example080_deepep_jit_dispatch_payload/nv/build_and_run.py:296-303) and the
kernels' real configuration is compile-time constants
(datasets/example051_thunderkitten_ag_gemm_easy/nv/empty_thunderkitten_ag_gemm.cu:86-99).
Here one dataclass holds the per-op tunables; the world size is a run-time value.
"""
from __future__ import annotations

import dataclasses
import os
from dataclasses import dataclass


@dataclass
class Config:
    # --- collectives -------------------------------------------------------
    ar_oneshot_max_bytes: int = 512 * 1024      # no multicast, at or below: one-shot pull all-reduce
    ar_nvls_min_bytes: int = 16                 # multicast bound, at or above: NVLS
    ar_nvls_max_bytes_two_ranks: int = 8 << 20  # with 2 ranks, NVLS only below this size
    coll_max_blocks: int = 64                   # CTAs per collective kernel (<= one wave)
    coll_max_blocks_large: int = 128            # bandwidth collectives of 16 MB and more
    ar_oneshot_grain_bytes: int = 8 * 1024      # message bytes per CTA, one-shot all-reduce
    ar_chunk_grain_bytes: int = 64 * 1024       # message bytes per CTA, two-shot / NVLS
    # --- fused GEMMs -------------------------------------------------------
    ag_gemm_comm_ctas: int = 8                  # CTAs reserved for pushing the local A shard
    gemm_ar_oneshot_max_m: int = 0              # rows at or below use the one-shot epilogue (0: never)
    gemm_ar_split_max_world: int = 4            # up to this many ranks "auto" runs GEMM + all-reduce as two launches
    fused_poll_ns: int = 300                    # GEMM->AR: pause between polls of a peer-written flag
    gemm_rs_poll_ns: int = 3000                 # GEMM->RS: pause between polls of a tile's arrival counter
    ag_gemm_row_poll_ns: int = 0                # AG->GEMM: pause between polls of a remote row block (0: back-off)
    ag_gemm_gate_poll_ns: int = 20000           # AG->GEMM: pause between polls of the host-copy gate
    # --- attention -------------------------------------------------------
    attn_impl: int = 4                          # flash-attention kernel: 4 (P kept in TMEM) or 1
    cp_comm_ctas: int = 4                       # ring attention: CTAs that pull the K/V shards
    cp_comm_ctas_ulysses: int = 16              # Ulysses: CTAs that pull the K/V head slices
    # --- MoE ---------------------------------------------------------------
    moe_fused_swiglu: bool = True               # silu(gate)*up in the up-projection's epilogue
    # --- runtime -----------------------------------------------------------
    heap_bytes: int = 1 << 30
    timeout_s: float = 2.0
    use_nvls: bool = True
    nvtx: bool = False                          # NVTX range around every op (external profilers)


_CONFIG: Config | None = None


def _coerce(value: str, typ):
    if typ is bool:
        return value.strip().lower() not in ("0", "false", "no", "off", "")
    return typ(value)


def get_config() -> Config:
    """The process-wide configuration (created on first use from the environment)."""
    global _CONFIG
    if _CONFIG is None:
        cfg = Config()
        for f in dataclasses.fields(Config):
            env = os.environ.get("CB200_" + f.name.upper())
            if env is not None:
                setattr(cfg, f.name, _coerce(env, type(getattr(cfg, f.name))))
        _CONFIG = cfg
    return _CONFIG


def set_config(**kw) -> Config:
    cfg = get_config()
    for k, v in kw.items():
        if not hasattr(cfg, k):
            raise KeyError(f"unknown config field {k!r}")
        setattr(cfg, k, v)
    return cfg


def reset_config():
    global _CONFIG
    _CONFIG = None
