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
    "nanosleep": {"info_only": True, "family": "utility", "examples": ["example076"]},
    "gpu_attributes": {"info_only": True, "family": "utility", "examples": ["example010"]},
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
    if e is None:
        return None
    if e == "info_only" or (isinstance(e, dict) and e.get("info_only")):
        return "info_only"
    return {"primary": e["primary"], "direction": e["direction"]}


def examples_covered() -> set[str]:
    out = set()
    for e in OPS.values():
        if isinstance(e, dict):
            out.update(e["examples"])
    return out


# Where each op lives in this package (what a user of the reference's example calls instead) and,
# where one is shipped, the generate/build/run task that poses the same exercise.
API: dict = {
    "all_reduce": ("ops.collectives.all_reduce (one-shot / two-shot / NVLS by size)",
                   "gloo_allreduce, oneshot_allreduce_virtual_ranks, nvls_all_reduce, "
                   "twoshot_allreduce_tuned"),
    "internode_all_reduce": ("ops.transport.PutSignalAllReduce", None),
    "all_gather": ("ops.collectives.all_gather (pull / push / multimem)",
                   "all_gather_last_dim, nvls_all_gather"),
    "reduce_scatter": ("ops.collectives.reduce_scatter (pull / multimem.ld_reduce)",
                       "reduce_scatter_blocks, nvls_reduce_scatter"),
    "all_to_all": ("ops.collectives.all_to_all, all_to_all_4d; ops.p2p.ulysses_all_to_all_nccl",
                   "ulysses_all_to_all, alltoall_4d_symmetric"),
    "broadcast": ("ops.collectives.broadcast; ops.p2p.WeightBroadcaster", "weight_broadcast"),
    "barrier": ("ops.collectives.barrier (flag matrix / multimem.red)", "nvls_barrier_latency"),
    "ag_gemm": ("ops.tp.AgGemm; parallel.tp.ColumnParallelLinear",
                "ag_gemm_fused, ag_gemm_fp8_fused, ag_gemm_virtual_ranks"),
    "gemm_rs": ("ops.tp.GemmRs; parallel.tp.RowParallelLinear",
                "gemm_rs_fused, gemm_rs_virtual_ranks"),
    "gemm_ar": ("ops.tp.GemmAr", "gemm_ar_fused"),
    "tp_qknorm": ("ops.fused.TPQKNorm", None),
    "gemm": ("ops.gemm.gemm, gemm_fp8_blockscaled", None),
    "moe_layer": ("ops.moe.MoELayer; parallel.ep.ExpertParallelMoE; ops.p2p.all_gatherv / reduce_scatterv",
                  "moe_agrs_dispatch, moe_dispatch_gemm"),
    "moe_dispatch_layout": ("ops.moe.dispatch_layout, router_topk, expert_sort", "moe_dispatch_layout"),
    "eplb_rebalance": ("ops.p2p.rearrange_expert_weights_inplace", "eplb_rebalance"),
    "ring_attention": ("ops.cp.RingAttention; parallel.cp.ContextParallelAttention",
                       "ring_attention_kernel"),
    "ulysses_attention": ("ops.cp.UlyssesAttention, ulysses_attention", "ulysses_attention_kernel"),
    "flash_attention": ("ops.cp.flash_attention", None),
    "p2p_copy": ("ops.util.peer_copy_bandwidth, memcpy_bandwidth, ipc_export / ipc_import", "d2d_copy_kernel"),
    "p2p_pingpong": ("ops.util.pingpong_latency", None),
    "put_signal": ("ops.shmem.put_signal", None),
    "get": ("ops.shmem.wait_get", None),
    "atomic_fetch_inc": ("ops.shmem.atomic_fetch_inc", "atomic_ticket_counter"),
    "tile_produce_consume": ("ops.shmem.tile_put, tile_consume", None),
    "pp_tensor_dict": ("ops.p2p.send_tensor_dict / recv_tensor_dict; parallel.pp.PipelineStage",
                       "tensor_dict_handoff"),
    "ipc_weight_handoff": ("ops.util.ipc_export / ipc_import", None),
    "d2h_fifo": ("ops.util.D2HFifo", None),
    "h2d_fifo": ("ops.util.H2DFifo", None),
    "shm_broadcast": ("ops.util.ShmBroadcast", "shm_object_broadcast"),
    "copy_widths": ("ops.util.copy_bandwidth", "d2d_copy_kernel"),
    "tma_stream": ("ops.util.tma_stream_bandwidth", "tma_bulk_copy_ring"),
    "mbarrier": ("ops.util.mbarrier_round_trip", "mbarrier_producer_consumer"),
    "nanosleep": ("ops.util.nanosleep_probe", "globaltimer_nanosleep"),
    "gpu_attributes": ("ops.util.device_attributes; harness.platform_detect", None),
    "rdma_transport": ("ops.transport (Context, Endpoint, MemoryRegion, MemoryPool, exchange_metadata)", None),
}

# Finer than per op where one op stands for many examples.
EXAMPLE_TASK: dict = {
    "example002": "rdma_rc_write_read", "example009": "rdma_rc_write_read",
    "example006": "rdma_tcp_exchange",
    "example008": "rdma_srq_write_imm", "example011": "rdma_srq_write_imm", "example013": "rdma_srq_write_imm",
    "example014": "rdma_inline_sgl", "example019": "rdma_inline_sgl",
    "example015": "rdma_memory_pool", "example016": "rdma_ud_datagram",
    "example024": "rdma_atomics", "example025": "rdma_atomics",
    "example026": "rdma_cq_overflow_event", "example027": "rdma_memory_window",
    "example021": "all_gather_last_dim", "example023": "reduce_scatter_blocks",
    "example038": "put_signal_virtual_ranks", "example096": "put_signal_virtual_ranks",
    "example039": "put_signal_virtual_ranks", "example090": "put_signal_virtual_ranks",
    "example032": "atomic_ticket_counter",
    "example022": "gloo_allreduce", "example105": "oneshot_allreduce_virtual_ranks",
    "example109": "oneshot_allreduce_virtual_ranks", "example020": "ulysses_all_to_all",
    "example058": "ulysses_attention_kernel", "example087": "weight_broadcast", "example084": "moe_agrs_dispatch",
    "example042": "moe_dispatch_layout", "example074": "d2d_copy_kernel", "example077": "d2d_copy_kernel",
    "example043": "nvls_all_reduce", "example048": "nvls_all_reduce", "example060": "nvls_all_reduce",
    "example045": "nvls_all_gather", "example046": "nvls_all_gather", "example059": "nvls_all_gather",
    "example050": "nvls_reduce_scatter", "example062": "nvls_reduce_scatter",
    "example091": "nvls_reduce_scatter", "example017": "nvls_barrier_latency",
    "example049": "alltoall_4d_symmetric", "example061": "alltoall_4d_symmetric",
    "example051": "ag_gemm_fused", "example063": "ag_gemm_fused",
    "example052": "ag_gemm_fp8_fused", "example064": "ag_gemm_fp8_fused",
    "example054": "gemm_rs_fused", "example066": "gemm_rs_fused",
    "example053": "gemm_ar_fused", "example065": "gemm_ar_fused",
    "example056": "moe_dispatch_gemm", "example068": "moe_dispatch_gemm",
    "example057": "ring_attention_kernel", "example069": "ring_attention_kernel",
    "example070": "ulysses_attention_kernel",
    "example031": "twoshot_allreduce_tuned", "example097": "twoshot_allreduce_tuned",
    "example004": "rdma_device_query", "example029": "rdma_device_query",
    "example007": "rdma_uc_write", "example028": "rdma_nic_clock",
    "example092": "transport_put_signal_allreduce",
    "example033": "put_signal_virtual_ranks", "example040": "put_signal_virtual_ranks",
    "example003": "fifo_device_host", "example005": "fifo_device_host",
    "example010": "gpu_attributes_probe", "example035": "tile_produce_consume",
    "example073": "p2p_pingpong", "example088": "ipc_weight_handoff",
    "example101": "tp_qknorm_virtual_ranks", "example102": "tp_qknorm_virtual_ranks",
}
EXAMPLE_API: dict = {
    "example004": "ops.transport.Context.device_info", "example029": "ops.transport.Context.device_info",
    "example028": "ops.transport.Context.clock_ns", "example007": "ops.transport (UC queue pairs, CUDA tensors as buffers)",
    "example015": "ops.transport.MemoryPool", "example006": "ops.transport.exchange_metadata",
}


def migration_table() -> str:
    """Markdown table: reference example -> op -> where it is in this package -> shipped task."""
    rows = []
    for op, e in OPS.items():
        api, task = API.get(op, ("", None))
        for ex in (e.get("examples", []) if isinstance(e, dict) else []):
            rows.append((ex, op, EXAMPLE_API.get(ex, api), EXAMPLE_TASK.get(ex, task) or "-"))
    lines = ["| reference example | op | in this package | shipped task |", "|---|---|---|---|"]
    lines += [f"| {ex} | {op} | `{api}` | {task} |" for ex, op, api, task in sorted(rows)]
    return "\n".join(lines) + "\n"


if __name__ == "__main__":
    print(migration_table(), end="")
