"""The thing to beat: the unfused NCCL (+ cuBLAS / PyTorch) composition of every op, run on
the same tensors in the same process.

Reference counterparts: the torch.distributed wrappers of datasets/example020...023
(``NcclAllToAll.Run``, ``NcclAllGather.all_gather_last_dim``, ``NcclAllReduce.Run``,
``NcclReduceScatter.run``), and the unfused GEMM + barrier + all-reduce sequence of
datasets/example053_thunderkitten_gemm_ar_easy.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def all_reduce(x: torch.Tensor) -> torch.Tensor:
    dist.all_reduce(x)
    return x


def all_gather(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    W = dist.get_world_size()
    if out is None:
        out = torch.empty((W * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x)
    return out


def reduce_scatter(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    W = dist.get_world_size()
    if out is None:
        out = torch.empty((x.shape[0] // W,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x)
    return out


def all_to_all(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    out = torch.empty_like(x) if out is None else out
    dist.all_to_all_single(out, x)
    return out


def ag_gemm(a_local: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.matmul(all_gather(a_local), b.t())


def gemm_rs(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return reduce_scatter(torch.matmul(a, b.t()))


def gemm_ar(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return all_reduce(torch.matmul(a, b.t()))


def moe_layer(x, topk_idx, topk_w, w1_local, w2_local, num_experts: int, I: int):
    """NCCL all-to-all dispatch (bf16) + per-expert cuBLAS GEMMs + all-to-all back + weighted
    index_add.  ``w1_local`` [El, 2I, H], ``w2_local`` [El, H, I]."""
    W = dist.get_world_size()
    T, H = x.shape
    K = topk_idx.shape[1]
    El = num_experts // W
    flat_e = topk_idx.reshape(-1).long()
    order = torch.sort(flat_e, stable=True).indices            # pairs sorted by global expert
    tok = order // K
    send = x[tok]
    counts = torch.bincount(flat_e, minlength=num_experts)
    send_splits = counts.view(W, El).sum(1)
    all_counts = torch.empty(W, num_experts, dtype=counts.dtype, device=x.device)
    dist.all_gather_into_tensor(all_counts, counts)
    rank = dist.get_rank()
    recv_counts = all_counts[:, rank * El:(rank + 1) * El]      # [src, local expert]
    recv_splits = recv_counts.sum(1)
    ss, rs = send_splits.tolist(), recv_splits.tolist()        # host sync: part of this baseline
    recv = torch.empty(sum(rs), H, dtype=x.dtype, device=x.device)
    dist.all_to_all_single(recv, send, rs, ss)
    # Rows arrive grouped by source, inside each source by expert: sort them ONCE by local expert,
    # run every expert on its contiguous slice (one grouped cuBLAS call where this torch has it,
    # otherwise one matmul per expert on slices whose bounds come from a single host read), and
    # undo the permutation.  No per-expert nonzero / gather / scatter.
    exp_of_row = torch.repeat_interleave(
        torch.arange(El, device=x.device).repeat(W), recv_counts.reshape(-1))
    perm = torch.sort(exp_of_row, stable=True).indices
    rows = recv[perm]
    per_expert = recv_counts.sum(0)
    offs = torch.cumsum(per_expert, 0).to(torch.int32)
    out_sorted = None
    if hasattr(torch, "_grouped_mm") and rows.shape[0] > 0:
        try:
            h1 = torch._grouped_mm(rows, w1_local.transpose(1, 2), offs=offs)
            sg = torch.nn.functional.silu(h1[:, :I]) * h1[:, I:]
            out_sorted = torch._grouped_mm(sg, w2_local.transpose(1, 2), offs=offs)
        except Exception:                                      # noqa: BLE001
            out_sorted = None
    if out_sorted is None:
        out_sorted = torch.empty(rows.shape[0], H, dtype=x.dtype, device=x.device)
        bounds = [0] + offs.tolist()
        for j in range(El):
            lo, hi = bounds[j], bounds[j + 1]
            if hi > lo:
                h1 = rows[lo:hi] @ w1_local[j].t()
                sg = torch.nn.functional.silu(h1[:, :I]) * h1[:, I:]
                out_sorted[lo:hi] = sg @ w2_local[j].t()
    out_rows = torch.empty_like(out_sorted)
    out_rows[perm] = out_sorted
    back = torch.empty(send.shape[0], H, dtype=x.dtype, device=x.device)
    dist.all_to_all_single(back, out_rows, ss, rs)
    y = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    y.index_add_(0, tok, back.float() * topk_w.reshape(-1)[order].unsqueeze(1))
    return y.to(x.dtype)


def ulysses_attention(q, k, v, causal: bool = True):
    """all_to_all_single exchanges + PyTorch scaled_dot_product_attention."""
    from ..ops.p2p import ulysses_all_to_all_nccl

    qh = ulysses_all_to_all_nccl(q, True)
    kh = ulysses_all_to_all_nccl(k, True)
    vh = ulysses_all_to_all_nccl(v, True)
    o = torch.nn.functional.scaled_dot_product_attention(
        qh.permute(0, 2, 1, 3), kh.permute(0, 2, 1, 3), vh.permute(0, 2, 1, 3), is_causal=causal,
        enable_gqa=True)
    return ulysses_all_to_all_nccl(o.permute(0, 2, 1, 3).contiguous(), False)
