"""Object broadcast from rank 0 to every other rank of one host through a ring buffer in POSIX
shared memory (no sockets on the data path).  Prints one JSON object.

Same exercise as the reference's datasets/example100_vllm_shm_broadcast_object (one writer,
``dequeue(timeout)`` on the readers, pickled payloads of 1 KiB to 1 MiB, :94-135,266-279), written
against ``mmap`` instead of a serving framework's queue class.

Launched as: torchrun --nproc-per-node W ref_shm_object_broadcast.py   (gloo only for the barriers)
"""
import json
import mmap
import os
import pickle
import struct
import time

import torch.distributed as dist

SIZES = [1 << 10, 16 << 10, 256 << 10, 1 << 20]
ROUNDS = 20
NSLOTS = 4
SLOT_BYTES = (1 << 20) + 4096
HEADER = 64                       # per slot: u64 sequence, u64 length, then one byte per reader


class MessageQueue:
    """Single writer, ``n_readers`` readers.  Slot i holds message number k with k % NSLOTS == i;
    its sequence word is k + 1 once the payload is complete; reader r sets byte 16 + r when done."""

    def __init__(self, path: str, n_readers: int, reader_index: int | None):
        self.n_readers, self.reader = n_readers, reader_index
        size = NSLOTS * (HEADER + SLOT_BYTES)
        if reader_index is None:
            fd = os.open(path, os.O_CREAT | os.O_RDWR | os.O_TRUNC, 0o600)
            os.ftruncate(fd, size)
        else:
            fd = os.open(path, os.O_RDWR)
        self.mem = mmap.mmap(fd, size)
        os.close(fd)
        self.next = 0

    def _slot(self, k: int) -> int:
        return (k % NSLOTS) * (HEADER + SLOT_BYTES)

    def enqueue(self, obj, timeout: float = 10.0):
        data = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
        if len(data) > SLOT_BYTES:
            raise ValueError("object too large for a slot")
        k, base = self.next, self._slot(self.next)
        deadline = time.monotonic() + timeout
        if k >= NSLOTS:             # the slot still holds message k - NSLOTS: every reader must be done
            while any(self.mem[base + 16 + r] == 0 for r in range(self.n_readers)):
                if time.monotonic() > deadline:
                    raise TimeoutError("readers did not drain the ring")
                time.sleep(0)
        self.mem[base + 16:base + 16 + self.n_readers] = bytes(self.n_readers)
        self.mem[base + HEADER:base + HEADER + len(data)] = data
        struct.pack_into("<Q", self.mem, base + 8, len(data))
        struct.pack_into("<Q", self.mem, base, k + 1)          # publish last
        self.next += 1

    def dequeue(self, timeout: float = 10.0):
        k, base = self.next, self._slot(self.next)
        deadline = time.monotonic() + timeout
        while struct.unpack_from("<Q", self.mem, base)[0] != k + 1:
            if time.monotonic() > deadline:
                raise TimeoutError(f"message {k} did not arrive")
            time.sleep(0)
        (n,) = struct.unpack_from("<Q", self.mem, base + 8)
        obj = pickle.loads(self.mem[base + HEADER:base + HEADER + n])
        self.mem[base + 16 + self.reader] = 1
        self.next += 1
        return obj

    def close(self):
        self.mem.close()


def payload(nbytes: int, i: int) -> dict:
    return {"step": i, "blob": bytes((i + j) % 251 for j in range(64)) * (nbytes // 64), "tag": f"m{i}"}


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    path = f"/dev/shm/cb_task_mq_{os.environ.get('MASTER_PORT', '0')}"
    q = None
    if rank == 0:
        q = MessageQueue(path, world - 1, None)
    dist.barrier()
    if rank != 0:
        q = MessageQueue(path, world - 1, rank - 1)
    ok, rows = True, []
    for n in SIZES:
        dist.barrier()
        t0 = time.perf_counter()
        for i in range(ROUNDS):
            if rank == 0:
                q.enqueue(payload(n, i))
            else:
                ok &= q.dequeue() == payload(n, i)
        dist.barrier()
        dt = (time.perf_counter() - t0) / ROUNDS
        rows.append({"data_size": n / 2**20, "latency_avg": dt * 1e6, "throughput_avg": n / dt / 1e9})
    if rank != 0:                                    # an empty queue must time out, not hang
        try:
            q.dequeue(timeout=0.05)
            ok = False
        except TimeoutError:
            pass
    flags = [None] * world
    dist.all_gather_object(flags, bool(ok))
    q.close()
    dist.barrier()
    if rank == 0:
        os.unlink(path)
        print(json.dumps({"Correctness": "PASS" if all(flags) else "FAIL", "data_size_unit": "MB",
                          "latency_unit": "us", "throughput_unit": "GB/s", "metrics": rows}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
