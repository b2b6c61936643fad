"""NCCL-side building blocks exercised on gloo / CPU ranks: tensor-dict hand-off, bucketed
weight broadcast, variable-size gather / reduce-scatter, EPLB rebalance, Ulysses exchange."""
import multiprocessing as mp
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))


def _worker(rank, world, port, case, q):
    import torch.distributed as dist

    from commbench_b200.ops import p2p

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok = True
    try:
        if case == "tensor_dict":
            # round-trip echo: rank 0 -> rank 1 -> rank 0, byte equality
            g = torch.Generator().manual_seed(1)
            d = {"hidden": torch.randn(33, 17, generator=g), "ids": torch.arange(50, dtype=torch.int64),
                 "empty": torch.empty(0), "step": 7, "name": "stage0",
                 **{f"t{i}": torch.randn(i + 1, generator=g).to(torch.bfloat16) for i in range(20)}}
            if rank == 0:
                p2p.send_tensor_dict(d, 1)
                back = p2p.recv_tensor_dict(1)
                for k, v in d.items():
                    if isinstance(v, torch.Tensor):
                        ok &= torch.equal(v, back[k]) and v.dtype == back[k].dtype
                    else:
                        ok &= back[k] == v
            elif rank == 1:
                got = p2p.recv_tensor_dict(0)
                p2p.send_tensor_dict(got, 0)
        elif case == "weights":
            names = [f"layer{i}.w" for i in range(10)]
            ref = {n: torch.randn(64 + i, 8, generator=torch.Generator().manual_seed(i))
                   for i, n in enumerate(names)}
            ref["scale"] = torch.arange(5, dtype=torch.int32)
            state = {n: (t.clone() if rank == 0 else torch.zeros_like(t)) for n, t in ref.items()}
            calls = p2p.WeightBroadcaster(src=0, bucket_bytes=4096).broadcast(state)
            ok &= calls >= 2
            ok &= all(torch.equal(state[n], ref[n]) for n in ref)
        elif case == "vcoll":
            sizes = [3 + 2 * r for r in range(world)]
            x = torch.full((sizes[rank], 4), float(rank + 1))
            g = p2p.all_gatherv(x, sizes)
            ref = torch.cat([torch.full((sizes[r], 4), float(r + 1)) for r in range(world)])
            ok &= torch.equal(g, ref)
            rs = p2p.reduce_scatterv(g * (rank + 1), sizes)
            tot = sum(r + 1 for r in range(world))
            ok &= torch.equal(rs, x * tot)
        elif case == "eplb":
            epr, layers = 2, 3
            nslots = world * epr
            old = list(range(nslots))
            new = [(s + 3) % nslots for s in range(nslots)]
            new[0] = old[0]                          # one slot keeps its expert
            new[1] = new[2]                          # a replicated (hot) expert
            def expert_weight(e, layer):
                return torch.full((5,), float(100 * layer + e))
            ws = [torch.stack([expert_weight(old[rank * epr + j], l) for j in range(epr)])
                  for l in range(layers)]
            p2p.rearrange_expert_weights_inplace(old, new, ws, epr)
            for l in range(layers):
                for j in range(epr):
                    ok &= torch.equal(ws[l][j], expert_weight(new[rank * epr + j], l))
        elif case == "ulysses":
            B, Sl, H, D = 2, 6, 4 * world, 8
            gen = torch.Generator().manual_seed(9)
            full = torch.randn(B, Sl * world, H, D, generator=gen)
            x = full[:, rank * Sl:(rank + 1) * Sl].contiguous()
            y = p2p.ulysses_all_to_all_nccl(x, to_heads=True)
            Hl = H // world
            ok &= torch.equal(y, full[:, :, rank * Hl:(rank + 1) * Hl].contiguous())
            z = p2p.ulysses_all_to_all_nccl(y, to_heads=False)
            ok &= torch.equal(z, x)                  # forward + inverse recovers the input
    except Exception as e:  # noqa: BLE001
        import traceback

        traceback.print_exc()
        ok = False
    dist.barrier()
    dist.destroy_process_group()
    q.put((rank, bool(ok)))


@pytest.mark.parametrize("case,world", [("tensor_dict", 2), ("weights", 2), ("vcoll", 3),
                                        ("eplb", 4), ("ulysses", 2)])
def test_p2p_blocks_on_gloo(case, world):
    from commbench_b200.runtime.launcher import free_port

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    ps = [ctx.Process(target=_worker, args=(r, world, port, case, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(world))
    for p in ps:
        p.join(60)
    assert all(res.values()), res
