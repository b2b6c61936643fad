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
  from the survivors, after which symmetric buffers are re-created on the new group.

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
        size = _HEADER + world * _SLOT.size
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

    # ------------------------------------------------------------------ peers
    def read(self, r: int) -> tuple[int, int, int, int]:
        return _SLOT.unpack_from(self.mm, _HEADER + r * _SLOT.size)

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

    def dead_ranks(self) -> list[int]:
        now = time.monotonic()
        dead = []
        for r in range(self.board.world):
            if r == self.board.rank:
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
