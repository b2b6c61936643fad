"""Registry of benchmarked ops: primary metric, direction, and the reference examples each op
stands in for.  Same role as ``PERF_METRICS`` in the reference (run_eval/perf_verdict.py:112-253:
one ``{primary, direction}`` entry or ``"info_only"`` per example), keyed by op instead of by
example directory.
"""
from __future__ import annotations

TIME = {"primary": "time_ms", "direction": "lower"}
BW = {"primary": "busbw_gbs", "direction": "higher"}

OPS: dict = {
    # ---- collectives --------------------------------------------------------------
    "all_reduce": {**TIME, "family": "collective",
                   "examples": ["example022", "example031", "example043", "example048", "example060",
                                "example095", "example097", "example098", "example099", "example105",
                                "example109"]},
    "internode_all_reduce": {**TIME, "family": "transport", "examples": ["example092"]},
    "all_gather": {**TIME, "family": "collective",
                   "examples": ["example021", "example030", "example045", "example046", "example059"]},
    "reduce_scatter": {**TIME, "family": "collective",
                       "examples": ["example023", "example037", "example050", "example062",
                                    "example091", "example093"]},
    "all_to_all": {**TIME, "family": "collective",
                   "examples": ["example018", "example020", "example044", "example049", "example061",
                                "example086"]},
    "broadcast": {**TIME, "family": "collective", "examples": ["example034", "example087"]},
    "barrier": {**TIME, "family": "collective", "examples": ["example017"]},
    # ---- fused tensor-parallel GEMMs --------------------------------------------------
    "ag_gemm": {**TIME, "family": "fusion", "examples": ["example051", "example052", "example063",
                                                         "example064"]},
    "gemm_rs": {**TIME, "family": "fusion", "examples": ["example054", "example055", "example066",
                                                         "example067"]},
    "gemm_ar": {**TIME, "family": "fusion", "examples": ["example053", "example065"]},
    "tp_qknorm": {**TIME, "family": "fusion", "examples": ["example101", "example102"]},
    "gemm": {**TIME, "family": "fusion", "examples": ["example053"]},
    # ---- expert parallel -----------------------------------------------------------------
    "moe_layer": {**TIME, "family": "ep", "examples": ["example056", "example068", "example078",
                                                       "example079", "example080", "example081",
                                                       "example082", "example083", "example084"]},
    "moe_dispatch_layout": {**TIME, "family": "ep", "examples": ["example042", "example047"]},
    "eplb_rebalance": {**TIME, "family": "ep", "examples": ["example089"]},
    # ---- context parallel ------------------------------------------------------------------
    "ring_attention": {**TIME, "family": "cp", "examples": ["example057", "example069"]},
    "ulysses_attention": {**TIME, "family": "cp", "examples": ["example058", "example070"]},
    "flash_attention": {**TIME, "family": "cp", "examples": []},
    # ---- point to point and utilities --------------------------------------------------------
    "p2p_copy": {**BW, "family": "p2p", "examples": ["example001", "example012", "example074"]},
    "p2p_pingpong": {**TIME, "family": "p2p", "examples": ["example073"]},
    "put_signal": {**BW, "family": "p2p", "examples": ["example033", "example038", "example040",
                                                       "example096"]},
    "get": {**BW, "family": "p2p", "examples": ["example039", "example090"]},
    "atomic_fetch_inc": {**TIME, "family": "p2p", "examples": ["example032"]},
    "tile_produce_consume": {**TIME, "family": "p2p", "examples": ["example035"]},
    "pp_tensor_dict": {**TIME, "family": "p2p", "examples": ["example085"]},
    "ipc_weight_handoff": {**TIME, "family": "p2p", "examples": ["example088"]},
    "d2h_fifo": {**TIME, "family": "utility", "examples": ["example003"]},
    "h2d_fifo": {**TIME, "family": "utility", "examples": ["example005"]},
    "shm_broadcast": {**TIME, "family": "utility", "examples": ["example100"]},
    "copy_widths": {**BW, "family": "utility", "examples": ["example075", "example077"]},
    "tma_stream": {**BW, "family": "utility", "examples": ["example094"]},
    "mbarrier": {**TIME, "family": "utility", "examples": ["example072"]},
    "nanosleep": "info_only",
    "gpu_attributes": "info_only",
    "rdma_transport": {**TIME, "family": "rdma",
                       "examples": ["example002", "example004", "example006", "example007",
                                    "example008", "example009", "example011", "example013",
                                    "example014", "example015", "example016", "example019",
                                    "example024", "example025", "example026", "example027",
                                    "example028", "example029"]},
}


def entry(op: str):
    """Registry entry of an op, or None when the op is unknown."""
    e = OPS.get(op)
    if e is None or e == "info_only":
        return e
    return {"primary": e["primary"], "direction": e["direction"]}


def examples_covered() -> set[str]:
    out = set()
    for e in OPS.values():
        if isinstance(e, dict):
            out.update(e["examples"])
    return out
