"""Mixture-of-experts token exchange built from two variable-size collectives: dispatch =
all-gather of every rank's tokens (ranks hold different numbers of tokens), combine =
reduce-scatter of the expert outputs back to the token owners.  Prints one JSON object.

Reference counterpart: datasets/example084_vllm_agrs_moe_all_to_all (dispatch as all_gatherv and
combine as reduce_scatterv with imbalanced per-rank sizes :104-173, sweep :347-352), here on CPU
tensors with the gloo backend so that it runs anywhere.

Launched as: torchrun --nproc-per-node W ref_moe_agrs_dispatch.py
"""
import json
import time

import torch
import torch.distributed as dist

HIDDEN = 512
MEAN_TOKENS = [64, 256, 1024]
ITERS = 3


def rank_sizes(mean: int, world: int) -> list[int]:
    """Imbalanced token counts, the same list on every rank (rank r: mean * (0.5 + r / (W - 1)))."""
    if world == 1:
        return [mean]
    return [max(1, int(mean * (0.5 + r / (world - 1)))) for r in range(world)]


class AgRsAll2All:
    def __init__(self):
        dist.init_process_group("gloo")
        self.rank, self.world = dist.get_rank(), dist.get_world_size()

    def dispatch(self, x: torch.Tensor, sizes: list[int]) -> torch.Tensor:
        """x [sizes[rank], H] -> [sum(sizes), H]: every rank's tokens in rank order."""
        # --- solution: an all-gather whose contributions differ in length (sizes is known on
        #     every rank; e.g. pad every contribution to max(sizes), gather, cut the padding off)
        mx = max(sizes)
        pad = torch.zeros(mx, x.shape[1], dtype=x.dtype)
        pad[:x.shape[0]] = x
        outs = [torch.empty_like(pad) for _ in sizes]
        dist.all_gather(outs, pad)
        return torch.cat([o[:n] for o, n in zip(outs, sizes)])
        # --- end solution

    def combine(self, y: torch.Tensor, sizes: list[int]) -> torch.Tensor:
        """y [sum(sizes), H] (this rank's partial outputs for ALL tokens) -> [sizes[rank], H]:
        the sum over ranks of the rows that belong to this rank's tokens."""
        # --- solution: a reduce-scatter with uneven slices (gloo has no reduce_scatter: e.g.
        #     all_reduce a copy and keep this rank's slice)
        full = y.clone()
        dist.all_reduce(full)
        return torch.split(full, sizes)[self.rank].clone()
        # --- end solution

    def close(self):
        dist.destroy_process_group()


def tokens_of(rank: int, n: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(1000 + rank)
    return torch.randint(-8, 9, (n, HIDDEN), generator=g).float()      # small integers: exact sums


def main():
    op = AgRsAll2All()
    r, W = op.rank, op.world
    ok, rows = True, []
    for mean in MEAN_TOKENS:
        sizes = rank_sizes(mean, W)
        x = tokens_of(r, sizes[r])
        allx = op.dispatch(x, sizes)
        want = torch.cat([tokens_of(q, sizes[q]) for q in range(W)])
        ok &= allx.shape == want.shape and torch.equal(allx, want)
        # every rank is the "expert" that scales tokens by (rank + 1); owners get the sum back
        back = op.combine(allx * (r + 1), sizes)
        ok &= torch.equal(back, x * (W * (W + 1) // 2))
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(ITERS):
            op.combine(op.dispatch(x, sizes) * (r + 1), sizes)
        dist.barrier()
        dt = (time.perf_counter() - t0) / ITERS
        nbytes = sum(sizes) * HIDDEN * 4
        rows.append({"data_size": nbytes / 2**20, "latency_avg": dt * 1e6, "throughput_avg": 2 * nbytes / dt / 1e9})
    flags = [None] * W
    dist.all_gather_object(flags, bool(ok))
    if r == 0:
        print(json.dumps({"Correctness": "PASS" if all(flags) else "FAIL", "data_size_unit": "MB",
                          "latency_unit": "us", "throughput_unit": "GB/s", "metrics": rows}))
    op.close()


if __name__ == "__main__":
    main()
