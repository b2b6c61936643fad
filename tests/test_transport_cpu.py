"""Loopback transport: the verbs-style patterns of the reference's RDMA examples
(example002 ... example029), each checked on host memory.  No NIC and no GPU needed."""
import socket
import threading

import numpy as np
import pytest

from commbench_b200.ops import transport as T


@pytest.fixture()
def ctx(native_lib):
    c = T.Context(T.LOOPBACK, "lo0")
    yield c
    c.close()


def _pair(ctx, qp_type=T.RC, **kw):
    a, b = ctx.create_qp(qp_type, **kw), ctx.create_qp(qp_type, **kw)
    T.connect_pair(a, b)
    return a, b


def test_device_info_is_deterministic(ctx):
    i1, i2 = ctx.device_info(), ctx.device_info()
    assert i1 == i2 and i1["backend"] == "loopback" and i1["atomic_cap"] == "ATOMIC_GLOB"
    assert i1["data_in_order"]["RC"]["WRITE"] is True and i1["data_in_order"]["UD"]["WRITE"] is False
    assert T.backend_available(T.LOOPBACK)
    t0 = ctx.clock_ns()
    assert ctx.clock_ns() >= t0


@pytest.mark.parametrize("nbytes", [64 << 10, 1 << 20])
def test_rc_write_read_send_recv(ctx, nbytes):
    a, b = _pair(ctx)
    src = np.random.default_rng(0).integers(0, 255, nbytes, dtype=np.uint8)
    dst = np.zeros(nbytes, dtype=np.uint8)
    ms, md = ctx.reg_mr(src), ctx.reg_mr(dst)
    a.post(T.WRITE, [ms.sge()], wr_id=1, remote_addr=md.addr, rkey=md.rkey)
    (c,) = a.poll_send()
    assert c.ok and c.wr_id == 1 and c.byte_len == nbytes and np.array_equal(src, dst)
    back = np.zeros(nbytes, dtype=np.uint8)
    mb = ctx.reg_mr(back)
    a.post(T.READ, [mb.sge()], wr_id=2, remote_addr=md.addr, rkey=md.rkey)
    assert a.poll_send()[0].ok and np.array_equal(back, src)
    # two-sided
    dst[:] = 0
    b.post_recv(7, [md.sge()])
    a.post(T.SEND, [ms.sge()], wr_id=3)
    rc = b.poll_recv()[0]
    assert rc.ok and rc.wr_id == 7 and rc.opcode == T.RECV and rc.byte_len == nbytes
    assert rc.src_qpn == a.qpn and np.array_equal(src, dst)
    assert a.poll_send()[0].wr_id == 3


def test_rc_send_waits_for_a_late_receive(ctx):
    a, b = _pair(ctx)
    src, dst = np.arange(64, dtype=np.uint8), np.zeros(64, dtype=np.uint8)
    ms, md = ctx.reg_mr(src), ctx.reg_mr(dst)
    a.post(T.SEND, [ms.sge()], wr_id=1)
    assert a.poll_send(timeout_us=1000) == []          # nothing completes until a receive exists
    b.post_recv(9, [md.sge()])
    assert b.poll_recv()[0].wr_id == 9 and a.poll_send()[0].ok and np.array_equal(src, dst)


def test_uc_send_recv_and_restrictions(ctx):
    a, b = _pair(ctx, T.UC)
    src, dst = np.full(256, 5, dtype=np.uint8), np.zeros(256, dtype=np.uint8)
    ms, md = ctx.reg_mr(src), ctx.reg_mr(dst)
    a.post(T.SEND, [ms.sge()], wr_id=1)                # no receive posted: lost, sender still completes
    assert a.poll_send()[0].ok and b.poll_recv(timeout_us=1000) == []
    b.post_recv(2, [md.sge()])
    a.post(T.SEND, [ms.sge()], wr_id=3)
    assert b.poll_recv()[0].ok and np.array_equal(src, dst)
    with pytest.raises(T.TransportError):
        a.post(T.READ, [md.sge()], remote_addr=ms.addr, rkey=ms.rkey)


def test_write_with_immediate_and_zero_byte_notification(ctx):
    a, b = _pair(ctx)
    src, dst = np.full(1024, 3, dtype=np.uint8), np.zeros(1024, dtype=np.uint8)
    ms, md = ctx.reg_mr(src), ctx.reg_mr(dst)
    b.post_recv(11, [])
    a.post(T.WRITE_IMM, [ms.sge()], wr_id=1, imm=0xABCD, remote_addr=md.addr, rkey=md.rkey)
    rc = b.poll_recv()[0]
    assert rc.opcode == T.RECV_IMM and rc.imm == 0xABCD and rc.wr_id == 11 and np.array_equal(src, dst)
    b.post_recv(12, [])
    a.post(T.WRITE_IMM, [], wr_id=2, imm=77, remote_addr=md.addr, rkey=md.rkey)   # pure doorbell
    rc = b.poll_recv()[0]
    assert rc.imm == 77 and rc.byte_len == 0
    assert [c.wr_id for c in a.poll_send()] == [1, 2]


def test_inline_send_and_limit(ctx):
    a, b = _pair(ctx, max_inline=128)
    assert a.max_inline == 128
    small, dst = np.arange(100, dtype=np.uint8), np.zeros(100, dtype=np.uint8)
    md = ctx.reg_mr(dst)
    addr, n = T.buffer_address(small)
    a.post(T.WRITE, [(addr, n, 0)], flags=T.SIGNALED | T.INLINE, remote_addr=md.addr, rkey=md.rkey)
    assert a.poll_send()[0].ok and np.array_equal(small, dst)     # no local key needed inline
    big = np.zeros(200, dtype=np.uint8)
    with pytest.raises(T.TransportError):
        a.post(T.WRITE, [(T.buffer_address(big)[0], 200, 0)], flags=T.INLINE, remote_addr=md.addr,
               rkey=md.rkey)


def test_scatter_gather_write(ctx):
    a, b = _pair(ctx)
    parts = [np.full(1000 + 10 * i, i + 1, dtype=np.uint8) for i in range(4)]
    mrs = [ctx.reg_mr(p) for p in parts]
    total = sum(p.size for p in parts)
    dst = np.zeros(total, dtype=np.uint8)
    md = ctx.reg_mr(dst)
    a.post(T.WRITE, [m.sge() for m in mrs], remote_addr=md.addr, rkey=md.rkey)
    assert a.poll_send()[0].byte_len == total and np.array_equal(dst, np.concatenate(parts))


def test_shared_receive_queue(ctx):
    srq, cq = ctx.create_srq(16), ctx.create_cq()
    r1 = ctx.create_qp(T.RC, send_cq=cq, recv_cq=cq, srq=srq)
    r2 = ctx.create_qp(T.RC, send_cq=cq, recv_cq=cq, srq=srq)
    s1, s2 = ctx.create_qp(T.RC), ctx.create_qp(T.RC)
    T.connect_pair(s1, r1)
    T.connect_pair(s2, r2)
    bufs = [np.zeros(32, dtype=np.uint8) for _ in range(2)]
    for i, bf in enumerate(bufs):
        ctx.post_srq_recv(srq, 100 + i, [ctx.reg_mr(bf).sge()])
    with pytest.raises(T.TransportError):
        r1.post_recv(1, [])                            # receives go to the shared queue
    m1, m2 = ctx.reg_mr(np.full(32, 1, dtype=np.uint8)), ctx.reg_mr(np.full(32, 2, dtype=np.uint8))
    s1.post(T.SEND, [m1.sge()])
    s2.post(T.SEND, [m2.sge()])
    got = sorted((c.qpn, c.wr_id) for c in ctx.poll_cq(cq) if c.opcode == T.RECV)
    assert got == sorted([(r1.qpn, 100), (r2.qpn, 101)])
    assert bufs[0][0] == 1 and bufs[1][0] == 2


def test_ud_datagrams(ctx):
    a, b = ctx.create_qp(T.UD), ctx.create_qp(T.UD)
    a.connect()
    b.connect()
    msg = np.arange(200, dtype=np.uint8)
    rbuf = np.zeros(T.UD_HEADER + 200, dtype=np.uint8)
    mm, mr = ctx.reg_mr(msg), ctx.reg_mr(rbuf)
    b.post_recv(1, [mr.sge()])
    a.post(T.SEND, [mm.sge()], dest=b.addr)
    c = b.poll_recv()[0]
    assert c.ok and c.byte_len == T.UD_HEADER + 200 and np.array_equal(rbuf[T.UD_HEADER:], msg)
    with pytest.raises(T.TransportError):              # one MTU at most
        a.post(T.SEND, [ctx.reg_mr(np.zeros(T.UD_MTU + 1, dtype=np.uint8)).sge()], dest=b.addr)
    with pytest.raises(T.TransportError):
        a.post(T.WRITE, [mm.sge()], dest=b.addr)
    wrong = T.Addr.unpack(b.addr.pack())
    wrong.qkey ^= 1
    b.post_recv(2, [mr.sge()])
    a.post(T.SEND, [mm.sge()], dest=wrong)             # wrong qkey: silently dropped
    assert b.poll_recv(timeout_us=1000) == []


def test_atomics_exactly_one_winner(ctx):
    a, b = _pair(ctx)
    c2, d2 = _pair(ctx)
    target = np.zeros(1, dtype=np.uint64)
    mt = ctx.reg_mr(target)
    olds = [np.zeros(1, dtype=np.uint64) for _ in range(2)]
    mo = [ctx.reg_mr(o) for o in olds]
    a.post(T.ATOMIC_CAS, [mo[0].sge()], remote_addr=mt.addr, rkey=mt.rkey, compare_add=0, swap=111)
    c2.post(T.ATOMIC_CAS, [mo[1].sge()], remote_addr=mt.addr, rkey=mt.rkey, compare_add=0, swap=222)
    assert a.poll_send()[0].ok and c2.poll_send()[0].ok
    assert sorted(int(o[0]) for o in olds) == [0, 111] and int(target[0]) == 111
    target[0] = 0
    a.post(T.ATOMIC_FADD, [mo[0].sge()], remote_addr=mt.addr, rkey=mt.rkey, compare_add=1)
    c2.post(T.ATOMIC_FADD, [mo[1].sge()], remote_addr=mt.addr, rkey=mt.rkey, compare_add=1)
    a.poll_send(), c2.poll_send()
    assert sorted(int(o[0]) for o in olds) == [0, 1] and int(target[0]) == 2
    a.post(T.ATOMIC_FADD, [mo[0].sge()], remote_addr=mt.addr + 4, rkey=mt.rkey, compare_add=1)
    assert a.poll_send()[0].status == T.REM_INV_REQ_ERR     # misaligned target


def test_remote_key_and_bounds_are_enforced(ctx):
    a, b = _pair(ctx)
    src, dst = np.ones(64, dtype=np.uint8), np.zeros(64, dtype=np.uint8)
    ms = ctx.reg_mr(src)
    ro = ctx.reg_mr(dst, T.LOCAL_WRITE | T.REMOTE_READ)
    a.post(T.WRITE, [ms.sge()], remote_addr=ro.addr, rkey=ro.rkey)
    assert a.poll_send()[0].status == T.REM_ACCESS_ERR and not dst.any()
    a.post(T.WRITE, [ms.sge()], wr_id=5, remote_addr=ro.addr, rkey=ro.rkey)
    assert a.poll_send()[0].status == T.WR_FLUSH_ERR          # the queue pair is dead after an error
    c, d = _pair(ctx)
    rw = ctx.reg_mr(dst)
    c.post(T.WRITE, [ms.sge()], remote_addr=rw.addr + 32, rkey=rw.rkey)   # runs past the end
    assert c.poll_send()[0].status == T.REM_ACCESS_ERR


def test_memory_window_bind_and_invalidate(ctx):
    a, b = _pair(ctx)
    region = np.zeros(4096, dtype=np.uint8)
    mr = ctx.reg_mr(region)
    mw = ctx.alloc_mw()
    with pytest.raises(T.TransportError):
        ctx.mw_rkey(mw)                                     # not bound yet
    b.post(T.BIND_MW, mw=mw, bind=(mr, 1024, 512, T.REMOTE_WRITE))
    assert b.poll_send()[0].ok
    wkey = ctx.mw_rkey(mw)
    src = np.full(512, 9, dtype=np.uint8)
    ms = ctx.reg_mr(src)
    a.post(T.WRITE, [ms.sge()], remote_addr=mr.addr + 1024, rkey=wkey)
    assert a.poll_send()[0].ok and region[1024:1536].all() and not region[:1024].any()
    c, d = _pair(ctx)
    c.post(T.WRITE, [ms.sge()], remote_addr=mr.addr + 2048, rkey=wkey)    # outside the window
    assert c.poll_send()[0].status == T.REM_ACCESS_ERR
    b.post(T.LOCAL_INV, mw=wkey)
    assert b.poll_send()[0].ok
    e, f = _pair(ctx)
    e.post(T.WRITE, [ms.sge()], remote_addr=mr.addr + 1024, rkey=wkey)
    assert e.poll_send()[0].status == T.REM_ACCESS_ERR          # the key is gone


def test_cq_overflow_raises_async_event(ctx):
    cq = ctx.create_cq(depth=2)
    a = ctx.create_qp(T.RC, send_cq=cq, recv_cq=cq)
    b = ctx.create_qp(T.RC)
    T.connect_pair(a, b)
    src, dst = np.ones(8, dtype=np.uint8), np.zeros(8, dtype=np.uint8)
    ms, md = ctx.reg_mr(src), ctx.reg_mr(dst)
    assert ctx.get_async_event(timeout_ms=10) is None
    t0 = ctx.clock_ns()
    for i in range(4):                                      # never polled: the third one overflows
        a.post(T.WRITE, [ms.sge()], wr_id=i, remote_addr=md.addr, rkey=md.rkey)
    ev = ctx.get_async_event(timeout_ms=1000)
    assert ev == (T.EVENT_CQ_ERR, cq) and ctx.clock_ns() - t0 < 1_000_000_000
    ctx.ack_async_event()
    with pytest.raises(T.TransportError):
        ctx.ack_async_event()
    assert len(ctx.poll_cq(cq)) == 2
    with pytest.raises(T.TransportError):
        ctx.poll_cq(cq, timeout_us=0)                       # drained and in error


def test_unsignaled_sends_complete_silently(ctx):
    a, b = _pair(ctx)
    src, dst = np.ones(8, dtype=np.uint8), np.zeros(8, dtype=np.uint8)
    ms, md = ctx.reg_mr(src), ctx.reg_mr(dst)
    a.post(T.WRITE, [ms.sge()], flags=0, remote_addr=md.addr, rkey=md.rkey)
    assert dst.all() and a.poll_send(timeout_us=1000) == []


def test_memory_pool_stack_allocator(ctx):
    pool = T.MemoryPool(ctx, np.zeros(1 << 16, dtype=np.uint8), align=256)
    s1 = pool.alloc(1000)
    s2 = pool.alloc(100)
    assert s1[0] % 256 == 0 and s2[0] == s1[0] + 1024 and s1[2] == s2[2] == pool.mr.lkey
    pool.release()
    assert pool.alloc(50)[0] == s2[0]
    pool.release(2)
    assert pool.used == 0
    with pytest.raises(T.TransportError):
        pool.alloc(1 << 20)


def test_two_contexts_and_tcp_metadata_exchange(native_lib):
    """Two adapters whose owners meet over TCP, then one writes into the other's buffer."""
    srv = socket.socket()
    srv.bind(("127.0.0.1", 0))
    srv.listen(1)
    port = srv.getsockname()[1]
    result = {}

    def server():
        with T.Context() as c:
            buf = np.zeros(128, dtype=np.uint8)
            mr = c.reg_mr(buf)
            qp = c.create_qp(T.RC)
            conn, _ = srv.accept()
            peer, _, _ = T.exchange_metadata(conn, qp.addr, mr.addr, mr.rkey)
            qp.connect(peer)
            qp.post_recv(1, [])
            rc = qp.poll_recv(timeout_us=5_000_000)
            result["imm"] = rc[0].imm if rc else None
            result["data"] = buf.copy()
            conn.close()

    th = threading.Thread(target=server)
    th.start()
    with T.Context() as c:
        qp = c.create_qp(T.RC)
        s = socket.create_connection(("127.0.0.1", port))
        peer, raddr, rkey = T.exchange_metadata(s, qp.addr)
        qp.connect(peer)
        src = np.arange(128, dtype=np.uint8)
        qp.post(T.WRITE_IMM, [c.reg_mr(src).sge()], imm=42, remote_addr=raddr, rkey=rkey)
        assert qp.poll_send()[0].ok
        s.close()
    th.join(10)
    srv.close()
    assert result["imm"] == 42 and np.array_equal(result["data"], np.arange(128, dtype=np.uint8))


def test_two_rank_allreduce_over_put_and_signal(ctx):
    a, b = _pair(ctx)
    ra, rb = T.PutSignalAllReduce(ctx, a, 1024), T.PutSignalAllReduce(ctx, b, 1024)
    ra.connect_window(rb.window())
    rb.connect_window(ra.window())
    rng = np.random.default_rng(3)
    for _ in range(3):
        xa, xb = rng.random(1024, dtype=np.float32), rng.random(1024, dtype=np.float32)
        ra.start(xa)
        rb.start(xb)
        ya, yb = ra.finish(), rb.finish()
        assert np.array_equal(ya, yb) and np.allclose(ya, xa + xb)
    lonely = T.PutSignalAllReduce(ctx, a, 8)
    lonely.connect_window(rb.window())
    lonely.start(np.ones(8, dtype=np.float32))
    with pytest.raises(T.TransportError, match="signal never arrived"):
        lonely.finish(timeout_s=0.3)                    # nobody answers: bounded wait, no hang


def test_verbs_backend_type_checks_against_the_public_interface():
    """No RDMA stack here: the libibverbs backend is at least compiled (syntax and types only)
    against a declarations-only copy of the public interface it uses."""
    import os
    import shutil
    import subprocess

    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no host compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    util = os.path.join(root, "commbench_b200", "csrc", "util")
    r = subprocess.run([gxx, "-std=c++17", "-fsyntax-only", "-Wall", "-Werror",
                        "-I", os.path.join(root, "tests", "stubs"), "-I", util,
                        "-I", os.path.join(root, "commbench_b200", "csrc"),
                        os.path.join(util, "transport_verbs.cc")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    # and without the header the file must fall back to the "not built" stub
    r = subprocess.run([gxx, "-std=c++17", "-fsyntax-only", "-Wall", "-Werror", "-I", util,
                        "-I", os.path.join(root, "commbench_b200", "csrc"),
                        os.path.join(util, "transport_verbs.cc")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
