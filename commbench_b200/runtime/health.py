"""Failure detection on the host: heart-beats in shared memory, a check before every launch,
and re-rendezvous of the survivors.

The kernels of this package never wait without a limit (a wait that runs out sets a status word
and returns), which bounds the damage of a missing peer to one time-out.  This module keeps a
missing peer from being *launched against* in the first place:

* every rank of a node bumps a counter in a small POSIX shared-memory board from a daemon
  thread (``HeartbeatBoard``), and marks itself ``LEAVING`` when it exits on purpose;
* ``Watchdog.check()`` - called between steps, before the next kernel launch - raises
  ``RankFailure`` naming the ranks whose counter stopped or whose process is gone;
* ``rerendezvous()`` builds a fresh ``torch.distributed`` group (new store, ranks renumbered)
  from the survivors, after which symmetric buffers are re-created on the new group;
* ``ElasticRunner`` packages the three into a step loop: a membership barrier on the board
  before every step, re-rendezvous when somebody is missing, a hook for the caller to rebuild
  what hangs on the group.

The reference has per-wait device time-outs and host-side process containment but neither
heart-beats nor recovery (DeepEP's ``timeout_while`` and ``gpu_barrier`` time-outs,
datasets/example080_deepep_dispatch_impl/empty_deepep_dispatch_impl.cu:73-75,122-143;
``PR_SET_PDEATHSIG`` and session kill in
datasets/example060_thunderkitten_all_reduce_hard/nv/empty_thunderkitten_all_reduce.cu:538-542 and
run_eval/compile_run.py:156-199); failures here are always made on the host - a rank that
raises, exits or stops beating - never by faulting a GPU.
"""
from __future__ import annotations

import mmap
import os
import struct
import threading
import time

ALIVE, LEAVING, FAILED = 1, 2, 3
_SLOT = struct.Struct("<QQQQ")        # counter, pid, state, last error code
_HEADER = 64


class RankFailure(RuntimeError):
    def __init__(self, dead: list[int], why: str = ""):
        super().__init__(f"ranks {dead} are gone{': ' + why if why else ''}")
        self.dead = dead


def _pid_alive(pid: int) -> bool:
    if pid <= 0:
        return False
    try:
        os.kill(pid, 0)
    except ProcessLookupError:
        return False
    except PermissionError:
        return True
    # A zombie still answers kill(0): look at its state.
    try:
        with open(f"/proc/{pid}/stat") as f:
            return f.read().rsplit(")", 1)[1].split()[0] != "Z"
    except OSError:
        return True


class HeartbeatBoard:
    """``world`` slots in ``/dev/shm/<name>``; rank ``rank`` owns one slot and beats into it."""

    def __init__(self, name: str, rank: int, world: int, interval_s: float = 0.05, create: bool | None = None):
        self.name, self.rank, self.world, self.interval = name, rank, world, interval_s
        self.path = os.path.join("/dev/shm", name)
        self._steps_at = _HEADER + world * _SLOT.size          # one u64 "next step" word per rank
        size = self._steps_at + world * 8
        if create is None:
            create = rank == 0
        if create:
            fd = os.open(self.path, os.O_CREAT | os.O_RDWR, 0o600)
            os.ftruncate(fd, size)
        else:
            deadline = time.time() + 30
            while True:
                try:
                    fd = os.open(self.path, os.O_RDWR)
                    if os.fstat(fd).st_size >= size:
                        break
                    os.close(fd)
                except FileNotFoundError:
                    pass
                if time.time() > deadline:
                    raise TimeoutError(f"heartbeat board {self.path} did not appear")
                time.sleep(0.01)
        self.mm = mmap.mmap(fd, size)
        os.close(fd)
        self._stop = threading.Event()
        self._count = 0
        self._write(ALIVE)
        self._thread = threading.Thread(target=self._beat, name=f"heartbeat-{rank}", daemon=True)
        self._thread.start()

    # ---------------------------------------------------------------- own slot
    def _write(self, state: int, err: int = 0):
        self._count += 1
        _SLOT.pack_into(self.mm, _HEADER + self.rank * _SLOT.size, self._count, os.getpid(), state, err)

    def _beat(self):
        while not self._stop.wait(self.interval):
            self._write(ALIVE)

    def leave(self, failed: bool = False, err: int = 0):
        """Announces a deliberate exit (or a failure the rank noticed itself) and stops beating."""
        self._stop.set()
        self._thread.join(1.0)
        self._write(FAILED if failed else LEAVING, err)

    def close(self, unlink: bool = False):
        self._stop.set()
        self._thread.join(1.0)
        try:
            self.mm.close()
        except (BufferError, ValueError):
            pass
        if unlink:
            try:
                os.unlink(self.path)
            except FileNotFoundError:
                pass

    def announce_step(self, step: int):
        """Publishes "this rank is about to run step ``step``" (see ``ElasticRunner``)."""
        struct.pack_into("<Q", self.mm, self._steps_at + self.rank * 8, step + 1)

    # ------------------------------------------------------------------ peers
    def read(self, r: int) -> tuple[int, int, int, int]:
        return _SLOT.unpack_from(self.mm, _HEADER + r * _SLOT.size)

    def step_of(self, r: int) -> int:
        """The step rank ``r`` last announced, -1 before its first announcement."""
        return struct.unpack_from("<Q", self.mm, self._steps_at + r * 8)[0] - 1

    def wait_all_present(self, timeout_s: float = 30.0):
        deadline = time.time() + timeout_s
        while any(self.read(r)[0] == 0 for r in range(self.world)):
            if time.time() > deadline:
                missing = [r for r in range(self.world) if self.read(r)[0] == 0]
                raise RankFailure(missing, "never joined")
            time.sleep(0.005)


class Watchdog:
    """Decides who is dead: a slot whose state is not ALIVE, whose process is gone, or whose
    counter has not moved for ``timeout_s``."""

    def __init__(self, board: HeartbeatBoard, timeout_s: float = 1.0):
        self.board, self.timeout = board, timeout_s
        now = time.monotonic()
        self._seen = {r: (board.read(r)[0], now) for r in range(board.world)}
        self.ignored: set[int] = set()      # ranks already dealt with (left out of later answers)

    def dead_ranks(self) -> list[int]:
        now = time.monotonic()
        dead = []
        for r in range(self.board.world):
            if r == self.board.rank or r in self.ignored:
                continue
            count, pid, state, _ = self.board.read(r)
            last_count, last_t = self._seen[r]
            if count != last_count:
                self._seen[r] = (count, now)
                last_t = now
            if state != ALIVE or not _pid_alive(pid) or now - last_t > self.timeout:
                dead.append(r)
        return dead

    def check(self):
        """Call between steps, with nothing in flight: raises instead of launching against a
        rank that is gone."""
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(dead)

    def wait_for_failure(self, timeout_s: float) -> list[int]:
        deadline = time.monotonic() + timeout_s
        while time.monotonic() < deadline:
            dead = self.dead_ranks()
            if dead:
                return dead
            time.sleep(self.board.interval)
        return []


def survivors_of(world: int, dead: list[int]) -> list[int]:
    return [r for r in range(world) if r not in set(dead)]


def rerendezvous(store_dir: str, old_rank: int, survivors: list[int], generation: int,
                 backend: str = "gloo", timeout_s: float = 30.0):
    """Tears the current default group down (if any) and joins a new one made of ``survivors``
    (old rank numbers); returns ``(new_rank, new_world)``.  Each generation uses its own
    file store, so stragglers of an older generation cannot interfere."""
    import datetime

    import torch.distributed as dist

    if old_rank not in survivors:
        raise RankFailure([old_rank], "this rank is not among the survivors")
    if dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:                      # noqa: BLE001 - the old group may be broken
            pass
    os.makedirs(store_dir, exist_ok=True)
    new_rank, new_world = sorted(survivors).index(old_rank), len(survivors)
    store = dist.FileStore(os.path.join(store_dir, f"generation{generation}"), new_world)
    dist.init_process_group(backend, store=store, rank=new_rank, world_size=new_world,
                            timeout=datetime.timedelta(seconds=timeout_s))
    return new_rank, new_world


class ElasticRunner:
    """A step loop that survives ranks leaving between steps.

    Before every step the members meet at a *membership barrier* on the heart-beat board: each
    announces the step it is about to run and waits until every other member has announced the
    same step - or has left, died or stopped beating.  Nobody therefore enters a collective with
    a rank that is not coming; when somebody is missing, the survivors tear the process group
    down, re-rendezvous under new rank numbers (``on_reconfigure(runner)`` lets the caller
    rebuild what hangs on the group: symmetric buffers, sharded state) and run the step as the
    smaller group.  The barrier costs a few shared-memory reads per step; nothing is in flight
    on a GPU while it runs.

        runner = ElasticRunner("job42", rank, world, "/tmp/job42/store").start()
        runner.run(lambda step, r: train_step(step, r.rank, r.world), steps=1000)
    """

    def __init__(self, name: str, rank: int, world: int, store_dir: str, backend: str = "gloo",
                 beat_s: float = 0.05, dead_after_s: float = 1.0, group_timeout_s: float = 30.0,
                 on_reconfigure=None):
        self.name, self.store_dir, self.backend = name, store_dir, backend
        self.first_rank, self.first_world = rank, world        # numbering on the board never changes
        self.rank, self.world = rank, world                    # numbering of the current group
        self.members = list(range(world))                      # board ranks still in the job
        self.generation = 0
        self.beat_s, self.dead_after_s, self.group_timeout_s = beat_s, dead_after_s, group_timeout_s
        self.on_reconfigure = on_reconfigure
        self.board: HeartbeatBoard | None = None
        self.watchdog: Watchdog | None = None
        self.history: list[dict] = []                          # one entry per reconfiguration

    def start(self) -> "ElasticRunner":
        self.board = HeartbeatBoard(self.name, self.first_rank, self.first_world, self.beat_s)
        self.board.wait_all_present()
        self.watchdog = Watchdog(self.board, self.dead_after_s)
        self.rank, self.world = rerendezvous(self.store_dir, self.first_rank, self.members, 0,
                                             self.backend, self.group_timeout_s)
        return self

    def membership_barrier(self, step: int, timeout_s: float = 60.0) -> list[int]:
        """Returns the members (board ranks) that will NOT take part in ``step``."""
        self.board.announce_step(step)
        deadline = time.monotonic() + timeout_s
        while True:
            dead = [r for r in self.watchdog.dead_ranks() if r in self.members]
            waiting = [r for r in self.members
                       if r != self.first_rank and r not in dead and self.board.step_of(r) < step]
            if not waiting:
                return dead
            if time.monotonic() > deadline:
                raise RankFailure(waiting, f"alive but never reached step {step}")
            time.sleep(min(self.beat_s, 0.005))

    def _reconfigure(self, dead: list[int], step: int):
        self.members = [r for r in self.members if r not in dead]
        self.watchdog.ignored.update(dead)
        self.generation += 1
        self.rank, self.world = rerendezvous(self.store_dir, self.first_rank, self.members,
                                             self.generation, self.backend, self.group_timeout_s)
        self.history.append({"step": step, "dead": list(dead), "world": self.world, "rank": self.rank})
        if self.on_reconfigure is not None:
            self.on_reconfigure(self)

    LEAVE = "leave"

    def run(self, step_fn, steps: int, first_step: int = 0):
        """Calls ``step_fn(step, runner)`` for every step; returns the number of steps run.  A
        ``step_fn`` that returns ``ElasticRunner.LEAVE`` has finished its last step: the rank
        announces its departure and the loop ends (a rank may only go between steps)."""
        for step in range(first_step, first_step + steps):
            dead = self.membership_barrier(step)
            if dead:
                self._reconfigure(dead, step)
            if step_fn(step, self) == self.LEAVE:
                self.leave()
                return step - first_step + 1
        return steps

    def leave(self, failed: bool = False):
        """Leaves the job between steps (nothing in flight): the others see it at their next
        membership barrier.  The process group is left as it is: the survivors abandon it."""
        self.board.leave(failed=failed)

    def close(self):
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
        self.board.close(unlink=(self.first_rank == min(self.members)))
