"""Child-process bodies of the failure-detection tests (run with ``python health_cases.py <case>
<rank> <world> <scratch dir>``).  Failures are made on the host only: a rank exits between
steps, announces nothing, or stops beating; nothing here faults or hangs a GPU."""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _report(scratch, rank, **kw):
    with open(os.path.join(scratch, f"result_rank{rank}.json"), "w") as f:
        json.dump(kw, f)


def cpu_elastic(rank, world, scratch, silent_exit):
    """Three gloo ranks all-reduce; the last one leaves between steps (announced, or silently);
    the others notice before their next collective, re-rendezvous and go on as two."""
    import torch
    import torch.distributed as dist

    from commbench_b200.runtime import health as H

    board = H.HeartbeatBoard(f"cb_health_{os.path.basename(scratch)}", rank, world, interval_s=0.02)
    board.wait_all_present()
    H.rerendezvous(os.path.join(scratch, "store"), rank, list(range(world)), generation=0)
    x = torch.full((4,), float(rank + 1))
    dist.all_reduce(x)
    step1 = x[0].item()
    dist.barrier()
    wd = H.Watchdog(board, timeout_s=0.5)
    if rank == world - 1:
        # Leaves between steps with nothing in flight.
        if silent_exit:
            board._stop.set()              # no announcement: the beat just stops
            time.sleep(0.1)
            os._exit(0)
        board.leave()
        _report(scratch, rank, step1=step1, left=True)
        return
    dead = wd.wait_for_failure(5.0)
    try:
        wd.check()
        raised = False
    except H.RankFailure as e:
        raised = e.dead == dead
    new_rank, new_world = H.rerendezvous(os.path.join(scratch, "store"), rank,
                                         H.survivors_of(world, dead), generation=1)
    y = torch.full((4,), float(rank + 1))
    dist.all_reduce(y)
    _report(scratch, rank, step1=step1, dead=dead, raised=raised, new_rank=new_rank,
            new_world=new_world, step2=y[0].item())
    dist.destroy_process_group()
    board.close(unlink=(rank == 0))


def gpu_leave(rank, world, scratch):
    """Two GPU ranks run a symmetric-memory all-reduce; rank 1 then leaves between steps.  Rank 0
    learns of it from the heart-beat board and raises instead of launching the next step.
    Multicast is off in this package and in NCCL, kernels use plain peer loads."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["CB200_NVLS"] = "0"
    import torch
    import torch.distributed as dist

    from commbench_b200.ops import collectives as coll
    from commbench_b200.runtime import health as H
    from commbench_b200.runtime.context import CommContext

    torch.cuda.set_device(rank)
    store = dist.FileStore(os.path.join(scratch, "pg"), world)
    dist.init_process_group("nccl", store=store, rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    board = H.HeartbeatBoard(f"cb_health_{os.path.basename(scratch)}", rank, world, interval_s=0.02)
    board.wait_all_present()
    ctx = CommContext(heap_bytes=64 << 20, use_multicast=False)
    x, _ = ctx.empty((1 << 16,), torch.bfloat16)
    x.fill_(rank + 1)
    out = torch.empty_like(x)
    coll.all_reduce(ctx, x, out=out, algo="oneshot")
    torch.cuda.synchronize()
    ctx.check_status()
    step1 = out[0].item()
    ctx.host_barrier()                      # both ranks are between steps, nothing in flight
    wd = H.Watchdog(board, timeout_s=0.5)
    if rank == 1:
        board.leave()
        _report(scratch, rank, step1=step1, left=True)
        torch.cuda.synchronize()
        os._exit(0)                         # no collective tear-down with a peer that stays
    dead = wd.wait_for_failure(10.0)
    launched = False
    try:
        wd.check()
        coll.all_reduce(ctx, x, out=out, algo="oneshot")   # must not be reached
        launched = True
    except H.RankFailure:
        pass
    torch.cuda.synchronize()
    _report(scratch, rank, step1=step1, dead=dead, launched=launched,
            status=int(ctx.status_word()))
    os._exit(0)


def cpu_runner(rank, world, scratch, silent_exit):
    """Four gloo ranks run eight all-reduce steps under ``ElasticRunner``; rank 3 leaves before
    step 3 and rank 1 before step 6 (announced, or by just exiting).  Every step's sum must be
    the number of members that took part in it."""
    import torch
    import torch.distributed as dist

    from commbench_b200.runtime import health as H

    seen = []
    runner = H.ElasticRunner(f"cb_runner_{os.path.basename(scratch)}", rank, world,
                             os.path.join(scratch, "store"), beat_s=0.02, dead_after_s=0.5,
                             on_reconfigure=lambda r: seen.append((r.generation, r.rank, r.world)))
    runner.start()
    sums = []

    def step_fn(step, r):
        x = torch.ones(8)
        dist.all_reduce(x)
        sums.append(int(x[0].item()))
        if (rank == 3 and step == 2) or (rank == 1 and step == 5):     # last step of this rank
            _report(scratch, rank, sums=sums, left_after=step)
            if silent_exit:
                os._exit(0)                    # no announcement at all: the beat just stops
            return r.LEAVE

    ran = runner.run(step_fn, steps=8)
    if ran < 8:
        os._exit(0)                            # left on purpose; the survivors keep the board
    _report(scratch, rank, sums=sums, reconfigured=seen, history=runner.history,
            members=runner.members, final=(runner.rank, runner.world))
    runner.close()


if __name__ == "__main__":
    case, rank, world, scratch = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    if case == "cpu_runner":
        cpu_runner(rank, world, scratch, silent_exit=False)
    elif case == "cpu_runner_silent":
        cpu_runner(rank, world, scratch, silent_exit=True)
    elif case == "cpu_elastic":
        cpu_elastic(rank, world, scratch, silent_exit=False)
    elif case == "cpu_elastic_silent":
        cpu_elastic(rank, world, scratch, silent_exit=True)
    elif case == "gpu_leave":
        gpu_leave(rank, world, scratch)
    else:
        raise SystemExit(f"unknown case {case}")
