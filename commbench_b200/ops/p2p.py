"""Point-to-point and library-collective building blocks that stay on NCCL:

* ``send`` / ``recv`` on a side stream (overlappable with compute)
* ``send_tensor_dict`` / ``recv_tensor_dict``: pipeline-parallel stage hand-off (metadata over
  the CPU group, tensors over NCCL p2p) - datasets/example085_vllm_pp_send_recv_tensor_dict/nv/
  empty_vllm_pp_send_recv_tensor_dict.py:97-140
* ``WeightBroadcaster``: trainer -> inference weight sync by bucketed broadcast -
  datasets/example087_vllm_nccl_weight_transfer_engine/nv/empty_vllm_nccl_weight_transfer_engine.py:127-176
* ``all_gatherv`` / ``reduce_scatterv``: MoE dispatch / combine as variable-size collectives -
  datasets/example084_vllm_agrs_moe_all_to_all/nv/empty_vllm_agrs_moe_all_to_all.py:104-173
* ``rearrange_expert_weights_inplace``: EPLB expert rebalance by batched isend/irecv -
  datasets/example089_vllm_eplb_expert_rebalance/nv/empty_vllm_eplb_expert_rebalance.py:122-180
* ``ulysses_all_to_all_nccl``: the 4-D exchange through ``all_to_all_single`` -
  datasets/example020_torch_distributed_nccl_alltoall/empty_nccl_alltoall.py:67-89

All functions also run on the gloo backend with CPU tensors, which is how their logic is
tested without a GPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _side_stream(t: torch.Tensor):
    if not t.is_cuda:
        return None
    if not hasattr(_side_stream, "s"):
        _side_stream.s = {}
    dev = t.device.index
    if dev not in _side_stream.s:
        _side_stream.s[dev] = torch.cuda.Stream(device=t.device)
    return _side_stream.s[dev]


def send(t: torch.Tensor, dst: int, group=None, overlap: bool = True):
    """NCCL send; with ``overlap`` it runs on a side stream ordered after the current one."""
    s = _side_stream(t) if overlap else None
    if s is None:
        dist.send(t, dst, group=group)
        return None
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        dist.send(t, dst, group=group)
        ev = torch.cuda.Event()
        ev.record(s)
    t.record_stream(s)
    return ev


def recv(t: torch.Tensor, src: int, group=None, overlap: bool = True):
    s = _side_stream(t) if overlap else None
    if s is None:
        dist.recv(t, src, group=group)
        return None
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        dist.recv(t, src, group=group)
        ev = torch.cuda.Event()
        ev.record(s)
    t.record_stream(s)
    return ev


# ------------------------------------------------------------- tensor dict (PP)
def send_tensor_dict(d: dict, dst: int, group=None, cpu_group=None):
    """Metadata (keys, shapes, dtypes, non-tensor values) goes over the CPU group as one
    pickled object, tensors follow over the device group in key order."""
    meta, tensors = [], []
    for k, v in d.items():
        if isinstance(v, torch.Tensor):
            meta.append((k, "tensor", tuple(v.shape), v.dtype, v.device.type))
            tensors.append(v.contiguous())
        else:
            meta.append((k, "object", v))
    dist.send_object_list([meta], dst=dst, group=cpu_group or group)
    for t in tensors:
        if t.numel():
            dist.send(t, dst, group=group)


def recv_tensor_dict(src: int, device=None, group=None, cpu_group=None) -> dict:
    box = [None]
    dist.recv_object_list(box, src=src, group=cpu_group or group)
    out = {}
    for item in box[0]:
        if item[1] == "tensor":
            _, _, shape, dtype, devtype = item
            t = torch.empty(shape, dtype=dtype, device=device if device is not None else devtype)
            if t.numel():
                dist.recv(t, src, group=group)
            out[item[0]] = t
        else:
            out[item[0]] = item[2]
    return out


# -------------------------------------------------------------- weight transfer
class WeightBroadcaster:
    """Broadcasts a named state dict from ``src`` in size-bounded buckets (one flat buffer per
    bucket, so many small tensors cost one collective)."""

    def __init__(self, src: int = 0, bucket_bytes: int = 256 << 20, group=None):
        self.src, self.bucket_bytes, self.group = src, bucket_bytes, group

    def _buckets(self, named):
        cur, size = [], 0
        for name, t in named:
            nb = t.numel() * t.element_size()
            if cur and size + nb > self.bucket_bytes:
                yield cur
                cur, size = [], 0
            cur.append((name, t))
            size += nb
        if cur:
            yield cur

    def broadcast(self, state: dict) -> int:
        """In place on every rank's tensors; returns the number of collectives issued."""
        calls = 0
        by_dtype: dict = {}
        for name in sorted(state):
            by_dtype.setdefault(state[name].dtype, []).append((name, state[name]))
        for dtype, named in by_dtype.items():
            for bucket in self._buckets(named):
                flat = torch.cat([t.reshape(-1) for _, t in bucket])
                dist.broadcast(flat, src=self.src, group=self.group)
                calls += 1
                off = 0
                for _, t in bucket:
                    n = t.numel()
                    t.copy_(flat[off:off + n].view_as(t))
                    off += n
        return calls


# ------------------------------------------------------------ v-collectives (MoE)
def all_gatherv(x: torch.Tensor, sizes: list[int], group=None) -> torch.Tensor:
    """Concatenation of every rank's rows; rank r contributes ``sizes[r]`` rows."""
    if len(set(sizes)) == 1:
        outs = [torch.empty_like(x) for _ in sizes]
        dist.all_gather(outs, x.contiguous(), group=group)
        return torch.cat(outs, dim=0)
    # uneven: pad every contribution to the largest one, gather, cut the padding off again
    mx = max(sizes)
    pad = torch.zeros((mx,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    pad[:x.shape[0]] = x
    outs = [torch.empty_like(pad) for _ in sizes]
    dist.all_gather(outs, pad, group=group)
    return torch.cat([o[:n] for o, n in zip(outs, sizes)], dim=0)


def reduce_scatterv(x: torch.Tensor, sizes: list[int], group=None) -> torch.Tensor:
    """Inverse: ``x`` holds sum(sizes) rows; rank r receives the sum over ranks of its slice."""
    rank = dist.get_rank(group)
    parts = list(torch.split(x.contiguous(), sizes, dim=0))
    if dist.get_backend(group) == "gloo":          # gloo has no reduce_scatter
        full = x.contiguous().clone()
        dist.all_reduce(full, group=group)
        return torch.split(full, sizes, dim=0)[rank].clone()
    out = torch.empty_like(parts[rank])
    dist.reduce_scatter(out, parts, group=group)
    return out


# ------------------------------------------------------------------ EPLB rebalance
def rearrange_expert_weights_inplace(old_map: list[int], new_map: list[int],
                                     weights: list[torch.Tensor], experts_per_rank: int,
                                     group=None) -> int:
    """``old_map[slot]`` / ``new_map[slot]`` = logical expert held in a physical slot (slot s
    lives on rank s // experts_per_rank).  Moves every layer tensor in ``weights`` (each
    ``[experts_per_rank, ...]``, this rank's slots) so that the new placement holds, with one
    ``batch_isend_irecv``.  Returns the number of p2p operations this rank issued."""
    rank = dist.get_rank(group)
    lo = rank * experts_per_rank
    ops, stage = [], []
    holder = {}
    for s, e in enumerate(old_map):
        holder.setdefault(e, s)                   # first slot that already holds the expert
    for s in range(lo, lo + experts_per_rank):     # what I must receive
        e = new_map[s]
        if old_map[s] == e:
            continue
        src_slot = holder[e]
        src_rank = src_slot // experts_per_rank
        for w in weights:
            if src_rank == rank:
                stage.append((w, s - lo, w[src_slot - lo].clone()))
            else:
                buf = torch.empty_like(w[s - lo])
                ops.append(dist.P2POp(dist.irecv, buf, src_rank, group=group))
                stage.append((w, s - lo, buf))
    for s, e in enumerate(new_map):                # what others need from me
        dst_rank = s // experts_per_rank
        if dst_rank == rank or old_map[s] == e:
            continue
        src_slot = holder[e]
        if src_slot // experts_per_rank != rank:
            continue
        for w in weights:
            ops.append(dist.P2POp(dist.isend, w[src_slot - lo].contiguous(), dst_rank, group=group))
    if ops:
        for r in dist.batch_isend_irecv(ops):
            r.wait()
    for w, idx, buf in stage:                      # install only after every send was posted
        w[idx].copy_(buf)
    return len(ops)


# ----------------------------------------------------------- Ulysses through NCCL
def ulysses_all_to_all_nccl(x: torch.Tensor, to_heads: bool, group=None) -> torch.Tensor:
    """[B, S/W, H, D] -> [B, S, H/W, D] (``to_heads``) or back, with ``all_to_all_single``."""
    W = dist.get_world_size(group)
    if to_heads:
        B, Sl, H, D = x.shape
        t = x.reshape(B, Sl, W, H // W, D).permute(2, 0, 1, 3, 4).contiguous()
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t, group=group)
        return out.permute(1, 0, 2, 3, 4).reshape(B, W * Sl, H // W, D)
    B, S, Hl, D = x.shape
    Sl = S // W
    t = x.reshape(B, W, Sl, Hl, D).permute(1, 0, 2, 3, 4).contiguous()
    out = torch.empty_like(t)
    dist.all_to_all_single(out, t, group=group)
    return out.permute(1, 2, 0, 3, 4).reshape(B, Sl, W * Hl, D)
