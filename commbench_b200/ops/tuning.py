"""Launch-shape table of the collectives: grid size, vectors in flight per thread and
algorithm per (op, world size, message size).

The bandwidth kernels are bound by bytes in flight (a peer or multicast load takes a few
microseconds), and the best grid differs between 2, 4 and 8 ranks and between 1 MB and
256 MB.  Rather than hard-coding one guess, the package ships a table measured on B200 +
NVSwitch (``tuning_b200_nvswitch.json`` beside this file) and
``python -m commbench_b200.ops.tune`` re-measures it on the machine at hand
(the role NCCL's tuner plug-in / ``NCCL_ALGO`` play for the library baseline of
datasets/example019_torch_distributed_nccl_allreduce/empty_nccl_allreduce.py:35-70).

Table layout::

    {"world": {"8": {"all_reduce": [[max_bytes, {"algo": "nvls", "blocks": 96, "unroll": 8}],
                                     ...],   # ascending max_bytes; the last row has null
                     "all_gather": [...], ...}}}

``CB200_TUNE_TABLE=<path>`` replaces the shipped table; ``CB200_TUNE_TABLE=off`` disables it.
Explicit ``blocks=`` / ``unroll=`` / ``algo=`` arguments of an op always win over the table.
"""
from __future__ import annotations

import json
import os
from pathlib import Path

_SHIPPED = Path(__file__).with_name("tuning_b200_nvswitch.json")
_cache: dict | None = None
_cache_key: str | None = None


def _load() -> dict:
    global _cache, _cache_key
    key = os.environ.get("CB200_TUNE_TABLE", "")
    if _cache is not None and key == _cache_key:
        return _cache
    table: dict = {}
    if key.lower() != "off":
        path = Path(key) if key else _SHIPPED
        try:
            table = json.loads(path.read_text())
        except (OSError, ValueError):
            table = {}
    _cache, _cache_key = table, key
    return table


def reload() -> None:
    """Drops the cached table (after writing a new one, or changing CB200_TUNE_TABLE)."""
    global _cache
    _cache = None


def lookup(op: str, world: int, nbytes: int, variant: str | None = None) -> dict:
    """Row of the table for ``op`` at ``world`` ranks and ``nbytes`` (the op's own size
    convention), or {} when nothing is recorded.  ``variant`` selects a sub-table
    (``"all_reduce@symmetric"`` before ``"all_reduce"``)."""
    w = _load().get("world", {}).get(str(world))
    if not w:
        return {}
    rows = None
    if variant:
        rows = w.get(f"{op}@{variant}")
    if rows is None:
        rows = w.get(op)
    if not rows:
        return {}
    for max_bytes, row in rows:
        if max_bytes is None or nbytes <= max_bytes:
            return dict(row)
    return dict(rows[-1][1])


def make_rows(points: list[tuple[int, dict]]) -> list:
    """Turns measured (size, best row) points into table rows: the boundary between two
    measured sizes is their geometric mean; the last row is open-ended."""
    points = sorted(points, key=lambda p: p[0])
    rows = []
    for i, (size, row) in enumerate(points):
        if i + 1 < len(points):
            bound = int((size * points[i + 1][0]) ** 0.5)
        else:
            bound = None
        rows.append([bound, row])
    return rows


def merge_into(path: Path, world: int, ops: dict) -> dict:
    """Writes/updates the entries of one world size in the table file at ``path``."""
    try:
        table = json.loads(Path(path).read_text())
    except (OSError, ValueError):
        table = {}
    table.setdefault("world", {}).setdefault(str(world), {}).update(ops)
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    Path(path).write_text(json.dumps(table, indent=1, sort_keys=True) + "\n")
    reload()
    return table
