"""Expert load balancing: the placement of logical experts on physical slots changes, and every
rank must end up holding the weights of the experts its slots are now assigned - moving only
what has to move, with all point-to-point transfers of a layer batched, and in place.
Prints one JSON object.

Launched as: torchrun --nproc-per-node 4 ref_eplb_rebalance.py
"""
import json
import time

import torch
import torch.distributed as dist

CASES = [(2, 4, 256), (3, 8, 1024), (4, 8, 2048)]        # (layers, local experts, hidden)


def expert_weight(layer: int, expert: int, hidden: int, which: int) -> torch.Tensor:
    """The one true value of a logical expert's tensor (any rank can rebuild it for checking)."""
    g = torch.Generator().manual_seed(layer * 100003 + expert * 101 + which)
    return torch.randn(hidden, 8 + 8 * which, generator=g)


def placements(n_slots: int, case: int) -> tuple[list[int], list[int]]:
    """Old and new slot -> logical expert maps: a rotation plus a few swaps; some slots keep their
    expert, some experts move inside a rank, most move across ranks."""
    old = list(range(n_slots))
    new = [(s + 3 + case) % n_slots if s % 4 else s for s in old]       # every fourth slot stays
    seen, fixed = set(), []
    for e in new:                                                        # keep it a permutation
        while e in seen:
            e = (e + 1) % n_slots
        seen.add(e)
        fixed.append(e)
    return old, fixed


def rearrange_expert_weights_inplace(old_map, new_map, weights, per_rank, rank) -> int:
    """``old_map[slot]`` / ``new_map[slot]`` = logical expert in a physical slot (slot s lives on
    rank s // per_rank).  ``weights``: this rank's tensors of ONE layer, each [per_rank, ...].
    Moves rows so that the new placement holds; returns the number of p2p operations issued."""
    # TODO: for every local slot whose expert changes find the slot that held that
    #       expert before; local source: copy through a temporary (the source row may itself be
    #       overwritten); remote source: one irecv per tensor; for every remote slot that needs an
    #       expert this rank held: one isend per tensor; post everything with ONE
    #       dist.batch_isend_irecv, wait, and only then install the received rows
    raise NotImplementedError


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    ok, rows = True, []
    for case, (layers, per_rank, hidden) in enumerate(CASES):
        n_slots = per_rank * world
        old, new = placements(n_slots, case)
        lo = rank * per_rank
        held = [[torch.stack([expert_weight(l, old[s], hidden, k) for s in range(lo, lo + per_rank)])
                 for k in range(2)] for l in range(layers)]
        dist.barrier()
        t0 = time.perf_counter()
        n_ops = sum(rearrange_expert_weights_inplace(old, new, held[l], per_rank, rank) for l in range(layers))
        dist.barrier()
        dt = time.perf_counter() - t0
        for l in range(layers):
            for k in range(2):
                want = torch.stack([expert_weight(l, new[s], hidden, k) for s in range(lo, lo + per_rank)])
                ok &= torch.equal(held[l][k], want)
        moved_in = sum(1 for s in range(lo, lo + per_rank)
                       if new[s] != old[s] and old.index(new[s]) // per_rank != rank)
        moved_out = sum(1 for s in range(n_slots)
                        if s // per_rank != rank and new[s] != old[s] and old.index(new[s]) // per_rank == rank)
        ok &= n_ops == (moved_in + moved_out) * 2 * layers          # nothing moves that need not
        nbytes = (moved_in + moved_out) * layers * hidden * (8 + 16) * 4
        rows.append({"data_size": nbytes / 2**20, "latency_avg": dt * 1e6,
                     "throughput_avg": nbytes / dt / 1e9 if dt > 0 else 0.0})
    flags = [None] * world
    dist.all_gather_object(flags, bool(ok))
    if rank == 0:
        print(json.dumps({"Correctness": "PASS" if all(flags) else "FAIL", "data_size_unit": "MB",
                          "latency_unit": "us", "throughput_unit": "GB/s", "metrics": rows}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
