"""Two endpoints that know nothing of each other meet over a TCP socket, exchange what a peer
needs (queue pair address, buffer address, remote key), connect, and then move data one-sidedly
in both directions: the client writes into the server's buffer and reads it back.
Prints one JSON object.

Reference counterpart: datasets/example006_rdma_read_write_rc (TCP exchange of QpMetadata :67,
150-205, then RC write / read between two adapters), here on the package's verbs-style transport
with the two sides as threads of one process, each with its own transport context.
"""
import json
import socket
import struct
import threading
import time

import numpy as np

from commbench_b200.ops import transport as T

SIZES = [64 << 10, 1 << 20, 8 << 20]
ADDR_BYTES = len(T.Addr().pack())


def send_metadata(sock: socket.socket, addr: T.Addr, buf_addr: int, rkey: int):
    # --- solution: one message: the packed queue pair address, then buffer address (u64) and
    #     remote key (u32), little endian
    sock.sendall(addr.pack() + struct.pack("<QI", buf_addr, rkey))
    # --- end solution


def recv_metadata(sock: socket.socket) -> tuple[T.Addr, int, int]:
    # --- solution: read exactly ADDR_BYTES + 12 bytes (a TCP read may return less than asked
    #     for); ConnectionError when the peer closes early
    need, raw = ADDR_BYTES + 12, b""
    while len(raw) < need:
        part = sock.recv(need - len(raw))
        if not part:
            raise ConnectionError("peer closed during the exchange")
        raw += part
    buf_addr, rkey = struct.unpack("<QI", raw[ADDR_BYTES:])
    return T.Addr.unpack(raw[:ADDR_BYTES]), buf_addr, rkey
    # --- end solution


def server(listener: socket.socket, result: dict):
    """Owns the target buffer; serves one client; never touches the data path."""
    with T.Context() as ctx:
        buf = np.zeros(max(SIZES), dtype=np.uint8)
        mr = ctx.reg_mr(buf)
        qp = ctx.create_qp(T.RC)
        conn, _ = listener.accept()
        with conn:
            # --- solution: receive the client's metadata, send ours (qp.addr, mr.addr, mr.rkey),
            #     connect the queue pair to the client's address, tell the client with one byte
            #     (b"r") that this side is connected, then wait for the client's one-byte "done"
            #     message on the socket before leaving
            peer, _, _ = recv_metadata(conn)
            send_metadata(conn, qp.addr, mr.addr, mr.rkey)
            qp.connect(peer)
            conn.sendall(b"r")
            conn.recv(1)
            # --- end solution
        result["tail"] = buf[:16].copy()


def client(port: int) -> tuple[bool, list, np.ndarray]:
    ok, rows = True, []
    with T.Context() as ctx:
        src, back = np.zeros(max(SIZES), dtype=np.uint8), np.zeros(max(SIZES), dtype=np.uint8)
        ms, mb = ctx.reg_mr(src), ctx.reg_mr(back)
        qp = ctx.create_qp(T.RC)
        with socket.create_connection(("127.0.0.1", port)) as s:
            # --- solution: send our metadata (no buffer: 0, 0), receive the server's
            #     (peer, raddr, rkey), connect, and wait for the server's one-byte "connected"
            send_metadata(s, qp.addr, 0, 0)
            peer, raddr, rkey = recv_metadata(s)
            qp.connect(peer)
            if s.recv(1) != b"r":
                raise ConnectionError("server did not report ready")
            # --- end solution
            rng = np.random.default_rng(1)
            qp.post(T.WRITE, [ms.sge(0, 16)], remote_addr=raddr, rkey=rkey)      # untimed first touch
            ok &= bool(qp.poll_send(timeout_us=5_000_000))
            for n in SIZES:
                src[:n] = rng.integers(0, 256, n, dtype=np.uint8)
                back[:n] = 0
                t0 = time.perf_counter()
                qp.post(T.WRITE, [ms.sge(0, n)], wr_id=1, remote_addr=raddr, rkey=rkey)
                w = qp.poll_send(timeout_us=5_000_000)
                dt = time.perf_counter() - t0
                qp.post(T.READ, [mb.sge(0, n)], wr_id=2, remote_addr=raddr, rkey=rkey)
                r = qp.poll_send(timeout_us=5_000_000)
                ok &= bool(w) and w[0].ok and bool(r) and r[0].ok and np.array_equal(back[:n], src[:n])
                rows.append({"data_size": n / 2**20, "latency_avg": dt * 1e6, "throughput_avg": n / dt / 1e9})
            s.sendall(b"x")
        return ok, rows, src[:16].copy()


def main():
    listener = socket.socket()
    listener.bind(("127.0.0.1", 0))
    listener.listen(1)
    result = {}
    th = threading.Thread(target=server, args=(listener, result), daemon=True)
    th.start()
    ok, rows, head = client(listener.getsockname()[1])
    th.join(20)
    listener.close()
    ok &= (not th.is_alive()) and "tail" in result and np.array_equal(result["tail"], head)
    print(json.dumps({"Correctness": "PASS" if ok else "FAIL", "data_size_unit": "MB", "latency_unit": "us",
                      "throughput_unit": "GB/s", "metrics": rows}))


if __name__ == "__main__":
    main()
