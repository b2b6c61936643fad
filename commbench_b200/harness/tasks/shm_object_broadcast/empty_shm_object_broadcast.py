"""Object broadcast from rank 0 to every other rank of one host through a ring buffer in POSIX
shared memory (no sockets on the data path).  Prints one JSON object.

Launched as: torchrun --nproc-per-node W empty_shm_object_broadcast.py   (gloo only for the barriers)
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
        # TODO: the writer (reader_index None) creates the file at `path` with room for NSLOTS
        # slots of HEADER + SLOT_BYTES bytes, readers open it; map it as self.mem; self.next = 0.
        raise NotImplementedError

    def enqueue(self, obj, timeout: float = 10.0):
        # TODO: pickle `obj`; before re-using a slot wait (TimeoutError after `timeout` seconds)
        # until every reader has marked the previous message in it as read; clear the reader
        # marks, write payload and length, and publish the sequence word LAST.
        raise NotImplementedError

    def dequeue(self, timeout: float = 10.0):
        # TODO: wait (TimeoutError after `timeout` seconds) for the sequence word of the next
        # message, unpickle it, mark it read for this reader, return the object.
        raise NotImplementedError

    def close(self):
        # TODO: unmap.
        raise NotImplementedError


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
