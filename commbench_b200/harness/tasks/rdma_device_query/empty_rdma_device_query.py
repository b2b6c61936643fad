"""Query a transport device before using it: port state, MTU, limits (queue pairs, completion
queues, memory regions, scatter/gather entries, inline bytes), atomic capability and the
"data arrives in order" table per queue-pair type and operation - then size resources from the
answers instead of from constants.  Prints one JSON object.
"""
import json
import time

import numpy as np

from commbench_b200.ops import transport as T

ROUNDS = 2000


class DeviceProbe:
    def __init__(self, ctx: T.Context):
        self.ctx = ctx

    def limits(self) -> dict:
        """{"active": bool, "mtu": int, "max_sge": int, "max_inline": int, "atomics": bool,
        "write_in_order": {"RC": bool, "UC": bool, "UD": bool}} from the device's own answers."""
        # TODO: ctx.device_info() gives port_state, mtu, max_sge, max_inline, atomic_cap
        #       ("ATOMIC_NONE" means no atomics) and data_in_order[type]["WRITE"]
        raise NotImplementedError

    def widest_gather(self, ep: T.Endpoint, mr: T.MemoryRegion, piece: int) -> int:
        """Posts ONE send that gathers as many `piece`-byte fragments of `mr` as the device allows
        in a single work request and returns that fragment count."""
        # TODO: max_sge fragments (not one more), offsets 0, 2*piece, 4*piece, ...
        raise NotImplementedError


def main():
    ok, rows = True, []
    with T.Context(T.LOOPBACK, "lo0") as ctx:
        probe = DeviceProbe(ctx)
        lim = probe.limits()
        info = ctx.device_info()
        ok &= lim["active"] and lim["mtu"] == info["mtu"] and lim["max_sge"] == info["max_sge"]
        ok &= lim["atomics"] == (info["atomic_cap"] != "ATOMIC_NONE")
        ok &= lim["write_in_order"] == {t: info["data_in_order"][t]["WRITE"] for t in ("RC", "UC", "UD")}
        a, b = ctx.create_qp(T.RC), ctx.create_qp(T.RC)
        T.connect_pair(a, b)
        piece = 64
        src = np.arange(2 * piece * (lim["max_sge"] + 2), dtype=np.uint8)
        dst = np.zeros(piece * (lim["max_sge"] + 2), dtype=np.uint8)
        ms, md = ctx.reg_mr(src), ctx.reg_mr(dst)
        b.post_recv(1, [md.sge()])
        n = probe.widest_gather(a, ms, piece)
        got = b.poll_recv()
        ok &= n == lim["max_sge"] and bool(got) and got[0].ok and got[0].byte_len == n * piece
        want = np.concatenate([src[2 * i * piece:2 * i * piece + piece] for i in range(n)])
        ok &= np.array_equal(dst[:n * piece], want)
        try:                                              # one fragment more must be refused
            a.post(T.SEND, [ms.sge(2 * i * piece, piece) for i in range(n + 1)], wr_id=8)
            ok = False
        except T.TransportError:
            pass
        t0 = time.perf_counter()
        for _ in range(ROUNDS):
            probe.limits()
        dt = (time.perf_counter() - t0) / ROUNDS
        rows.append({"data_size": 1, "latency_avg": dt * 1e6, "throughput_avg": 1.0 / dt / 1e6})
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "query", "latency_unit": "us",
                      "throughput_unit": "Mquery/s", "metrics": rows}))


if __name__ == "__main__":
    main()
