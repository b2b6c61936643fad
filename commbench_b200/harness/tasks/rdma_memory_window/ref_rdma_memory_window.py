"""Memory windows: expose a sub-range of a registered region to a peer for a while.  Bind a
window with a work request, hand its key to the peer, let the peer write through it, check that
writes outside the window are refused, invalidate the key and check that it is dead.
Prints one JSON object.

Reference counterpart: datasets/example027_rdma_ibv_wr_bind (bind / local invalidate work requests
on registered memory :77-112), here on the package's verbs-style transport.
"""
import json
import time

import numpy as np

from commbench_b200.ops import transport as T

REGION = 1 << 20
ROUNDS = 100


class WindowOwner:
    """Owns a registered region and one memory window over part of it."""

    def __init__(self, ctx: T.Context, qp: T.Endpoint):
        self.ctx, self.qp = ctx, qp
        self.buf = np.zeros(REGION, dtype=np.uint8)
        self.mr = ctx.reg_mr(self.buf)
        # --- solution: allocate one memory window (self.mw)
        self.mw = ctx.alloc_mw()
        # --- end solution

    def bind(self, offset: int, length: int, access: int = T.REMOTE_WRITE) -> int:
        """Binds the window to [offset, offset + length) of the region; returns the remote key."""
        # --- solution: post a T.BIND_MW work request on self.qp (mw=self.mw,
        #     bind=(self.mr, offset, length, access)), wait for its completion (RuntimeError on
        #     failure), return ctx.mw_rkey(self.mw)
        self.qp.post(T.BIND_MW, mw=self.mw, bind=(self.mr, offset, length, access))
        got = self.qp.poll_send(timeout_us=2_000_000)
        if not got or not got[0].ok:
            raise RuntimeError("bind failed")
        return self.ctx.mw_rkey(self.mw)
        # --- end solution

    def invalidate(self, rkey: int):
        # --- solution: post a T.LOCAL_INV work request for that key (mw=rkey) and wait for it
        self.qp.post(T.LOCAL_INV, mw=rkey)
        got = self.qp.poll_send(timeout_us=2_000_000)
        if not got or not got[0].ok:
            raise RuntimeError("invalidate failed")
        # --- end solution


def try_write(ctx: T.Context, src: T.MemoryRegion, remote_addr: int, rkey: int) -> int:
    """Completion status of one write from a fresh connected queue pair (an access error kills
    the queue pair, so every probe gets its own)."""
    a, b = ctx.create_qp(T.RC), ctx.create_qp(T.RC)
    T.connect_pair(a, b)
    a.post(T.WRITE, [src.sge()], remote_addr=remote_addr, rkey=rkey)
    got = a.poll_send(timeout_us=2_000_000)
    a.destroy()
    b.destroy()
    return got[0].status if got else -1


def main():
    ok = True
    with T.Context(T.LOOPBACK, "lo0") as ctx:
        oq, pq = ctx.create_qp(T.RC), ctx.create_qp(T.RC)
        T.connect_pair(oq, pq)
        owner = WindowOwner(ctx, oq)
        payload = np.full(4096, 9, dtype=np.uint8)
        src = ctx.reg_mr(payload)
        try:
            ctx.mw_rkey(owner.mw)
            ok = False                                       # an unbound window has no key
        except T.TransportError:
            pass
        key = owner.bind(64 << 10, 8192)
        base = owner.mr.addr + (64 << 10)
        ok &= try_write(ctx, src, base, key) == T.OK
        ok &= bool((owner.buf[64 << 10:(64 << 10) + 4096] == 9).all()) and not owner.buf[:64 << 10].any()
        ok &= try_write(ctx, src, base + 8192, key) == T.REM_ACCESS_ERR          # past the window
        ok &= try_write(ctx, src, base + 8192 - 100, key) == T.REM_ACCESS_ERR    # straddles its end
        ok &= try_write(ctx, src, owner.mr.addr, key) == T.REM_ACCESS_ERR        # before it
        ok &= not owner.buf[(64 << 10) + 8192:].any()
        owner.invalidate(key)
        ok &= try_write(ctx, src, base, key) == T.REM_ACCESS_ERR                 # the key is dead
        t0 = time.perf_counter()
        for i in range(ROUNDS):                                  # rebinding moves the window
            k = owner.bind((i % 16) * 4096, 4096)
            owner.invalidate(k)
        dt = (time.perf_counter() - t0) / ROUNDS
        k = owner.bind(0, 4096)
        ok &= try_write(ctx, src, owner.mr.addr, k) == T.OK and bool((owner.buf[:4096] == 9).all())
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "B", "latency_unit": "us",
                      "throughput_unit": "Mops/s",
                      "metrics": [{"data_size": 4096, "latency_avg": dt * 1e6, "throughput_avg": 1.0 / (dt * 1e6)}]}))


if __name__ == "__main__":
    main()
