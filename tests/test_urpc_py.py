"""URPC through the Python binding: synchronous and asynchronous calls, an unknown function, a request that the
server never answers (timeout), statistics."""
import os
import time

import pytest


@pytest.fixture()
def rpc(tmp_path):
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    from umdk_b200 import urpc
    urpc.init(default_timeout_ms=2000)
    srv = urpc.Server()
    srv.register(1, lambda b: b[::-1])
    srv.register(2, lambda b: str(sum(b)).encode())
    ch = urpc.Channel(srv.ip, srv.port)
    yield urpc, srv, ch
    ch.close()
    srv.stop()
    urpc.uninit()


def test_sync_async_timeout(rpc):
    urpc, srv, ch = rpc
    assert ch.call(1, b"hello urpc") == b"cpru olleh"
    payload = bytes(range(256)) * 40
    assert ch.call(2, payload) == str(sum(payload)).encode()
    # asynchronous calls complete through poll, carrying the caller's context
    for i in range(8):
        ch.call_async(1, bytes([65 + i]) * 10, user_ctx=100 + i)
    got = {}
    deadline = time.monotonic() + 5
    while len(got) < 8 and time.monotonic() < deadline:
        for ev, ctx, status, data in ch.poll():
            assert ev == urpc.POLL_RSP and status == 0
            got[ctx] = data
        time.sleep(0.001)
    assert got == {100 + i: bytes([65 + i]) * 10 for i in range(8)}
    # a server that stops polling: the call times out on the client, later calls work again
    srv.paused = True
    with pytest.raises(urpc.UrpcError) as e:
        ch.call(1, b"x", timeout_ms=200)
    assert e.value.code == urpc.ERR_TIMEOUT
    srv.paused = False
    assert ch.call(1, b"ab") == b"ba"
    st = urpc.stats()
    assert st["calls"] >= 12 and st["timeouts"] >= 1 and st["requests_served"] >= 11


def test_secured_connection_seals_payloads_and_refuses_other_keys(tmp_path):
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    from umdk_b200 import urpc
    key = "5c" * 32
    urpc.set_psk(key, "rpc")
    urpc.init(default_timeout_ms=2000)
    srv = urpc.Server()
    try:
        srv.register(1, lambda b: b[::-1])
        ch = urpc.Channel(srv.ip, srv.port)
        big = bytes(range(256)) * 100
        assert ch.call(1, b"sealed") == b"delaes" and ch.call(1, big) == big[::-1]
        rep = urpc.admin_query("sessions")
        assert "TLS_AES_256_GCM_SHA384" in rep and "payload sealed" in rep
        for bad_key, ident in (("6d" * 32, "rpc"), (key, "nobody"), ("", "")):
            urpc.set_psk(bad_key, ident)
            with pytest.raises(urpc.UrpcError):
                urpc.Channel(srv.ip, srv.port)
        urpc.set_psk(key, "rpc")
        assert ch.call(1, b"still works") == b"skrow llits"
        ch.close()
    finally:
        srv.stop()
        urpc.uninit()
        urpc.set_psk("", "")


def test_perf_recorder_sees_every_point(rpc):
    urpc, srv, ch = rpc
    got = {}
    urpc.perf_recorder(lambda point, ns: got.setdefault(point, []).append(ns))
    try:
        for _ in range(5):
            assert ch.call(1, b"abc") == b"cba"
    finally:
        urpc.perf_recorder(None)
    assert set(got) == set(urpc.PERF_POINTS)
    assert all(len(v) >= 5 for v in got.values())
    assert min(got["call_to_response"]) >= min(got["func_exec"])


def test_names_local_exec_channel_config_and_queue_reports(rpc):
    import ctypes
    urpc, srv, ch = rpc
    lib = urpc._lib()
    # a name for function 1, looked up by the client over its channel
    assert lib.urpc_func_name_register(ctypes.c_uint64(1), b"reverse") == 0
    assert lib.urpc_func_name_register(ctypes.c_uint64(77), b"nothing") != 0          # not registered
    lib.urpc_func_id_get.restype = ctypes.c_uint64
    assert lib.urpc_func_id_get(ch.id, b"reverse") == 1 and lib.urpc_func_id_get(ch.id, b"unknown") == 0
    # the same handler run in this process
    arg = ctypes.create_string_buffer(b"local", 5)
    sge = urpc._Sge(ctypes.cast(arg, ctypes.c_void_p), 5)
    rsp, rlen = ctypes.create_string_buffer(64), ctypes.c_uint32(64)
    assert lib.urpc_func_exec(ctypes.c_uint64(1), ctypes.byref(sge), 1, rsp, ctypes.byref(rlen)) == 0
    assert rsp.raw[:rlen.value] == b"lacol"
    assert lib.urpc_func_exec(ctypes.c_uint64(99), ctypes.byref(sge), 1, rsp, ctypes.byref(rlen)) != 0

    cfg = urpc._ChannelCfg()
    assert lib.urpc_channel_cfg_get(ch.id, ctypes.byref(cfg)) == 0
    assert cfg.attached == 1 and cfg.lost == 0 and cfg.server_port == srv.port and cfg.timeout_ms == 2000
    cfg.timeout_ms = 150
    assert lib.urpc_channel_cfg_set(ch.id, ctypes.byref(cfg)) == 0
    srv.paused = True
    t0 = time.monotonic()
    with pytest.raises(urpc.UrpcError):
        ch.call(1, b"x")                       # the channel's own timeout applies
    assert time.monotonic() - t0 < 1.0
    srv.paused = False
    # refresh = a new connection to the same server; calls keep working and an event reports it
    assert lib.urpc_channel_server_refresh(ch.id) == 0
    assert ch.call(1, b"again") == b"niaga"

    class Event(ctypes.Structure):
        _fields_ = [("type", ctypes.c_int), ("chid", ctypes.c_uint32), ("detail", ctypes.c_int)]
    ev = (Event * 4)()
    n = lib.urpc_async_event_get(ev, 4)
    assert n >= 1 and any(ev[i].type == 2 and ev[i].chid == ch.id for i in range(n))
    qh = (ctypes.c_uint64 * 1)()
    assert lib.urpc_channel_queue_query(ch.id, qh, 1) == 1
    status = ctypes.c_int(-1)
    assert lib.urpc_queue_status_query(ctypes.c_uint64(qh[0]), ctypes.byref(status)) == 0 and status.value == 1
    st = (ctypes.c_uint64 * 4)()
    assert lib.urpc_queue_stats_get(ctypes.c_uint64(qh[0]), st, 4) == 4 and st[0] >= 1 and st[2] >= 1
    lib.urpc_queue_stats_name_get.restype = ctypes.c_char_p
    assert lib.urpc_queue_stats_name_get(0) == b"tx_msgs" and lib.urpc_queue_stats_name_get(9) is None
    err = (ctypes.c_uint64 * 3)()
    assert lib.urpc_error_stats_get(err, 3) == 3 and err[1] >= 1            # the timeout above
    assert lib.urpc_hdr_size_get(0, 0) == 32
    msgs = (urpc._PollMsg * 4)()
    t0 = time.monotonic()
    assert lib.urpc_func_poll_wait(ch.id, msgs, 4, 100) == 0 and time.monotonic() - t0 >= 0.09


def test_arguments_by_reference(rpc):
    """A megabyte of client memory travels as a 90-byte description; the handler pulls it with one-sided reads."""
    import ctypes
    import zlib
    urpc, srv, ch = rpc
    seen = {}

    def checksum(args: bytes) -> bytes:
        seen["inline"], seen["refs"] = args, urpc.ref_count()
        try:
            head = urpc.ref_read(0, 0, 16)
            body = urpc.ref_read(0)
        except urpc.UrpcError as e:
            return b"ERR %d" % e.code
        return head + str(zlib.crc32(body)).encode()
    srv.register(5, checksum)
    n = 1 << 20
    mem = (ctypes.c_uint8 * n)(*([i * 7 & 0xff for i in range(4096)] * (n // 4096)))
    h = urpc.register_memory(ctypes.addressof(mem), n)
    out = ch.call_ref(5, b"crc", [(h, ctypes.addressof(mem), n)])
    assert seen == {"inline": b"crc", "refs": 1}
    assert out == bytes(mem[:16]) + str(zlib.crc32(bytes(mem))).encode()
    # a window of the registered memory; a window outside it is refused before anything is sent
    out = ch.call_ref(5, b"", [(h, ctypes.addressof(mem) + 4096, 8192)])
    assert out == bytes(mem[4096:4112]) + str(zlib.crc32(bytes(mem[4096:4096 + 8192]))).encode()
    with pytest.raises(urpc.UrpcError):
        ch.call_ref(5, b"", [(h, ctypes.addressof(mem) + n - 8, 64)])
    # remote access switched off: the call is refused; an ordinary call still shows no references
    lib = urpc._lib()
    assert lib.urpc_mem_seg_remote_access_disable(ctypes.c_uint64(h)) == 0
    with pytest.raises(urpc.UrpcError):
        ch.call_ref(5, b"", [(h, ctypes.addressof(mem), 64)])
    assert lib.urpc_mem_seg_remote_access_enable(ctypes.c_uint64(h)) == 0
    assert ch.call_ref(5, b"", [(h, ctypes.addressof(mem), 64)])[:16] == bytes(mem[:16])
    assert ch.call(5, b"plain").startswith(b"ERR") and seen["refs"] == 0
    urpc.unregister_memory(h)


def test_explicit_queue_given_to_a_channel(rpc):
    """A queue created on its own serves a channel that takes it before attaching; it survives the channel."""
    import ctypes
    urpc, srv, ch0 = rpc
    lib = urpc._lib()

    class QCfg(ctypes.Structure):
        _fields_ = [("rx_depth", ctypes.c_uint32), ("tx_depth", ctypes.c_uint32), ("rx_buf_size", ctypes.c_uint32),
                    ("interrupt", ctypes.c_int)]
    lib.urpc_queue_create.restype = ctypes.c_uint64
    qh = lib.urpc_queue_create(ctypes.byref(QCfg(32, 32, 16384, 0)))
    assert qh
    got = QCfg()
    assert lib.urpc_queue_cfg_get(ctypes.c_uint64(qh), ctypes.byref(got)) == 0 and got.rx_depth == 32
    assert lib.urpc_queue_cfg_set(ctypes.c_uint64(qh), ctypes.byref(QCfg(64, 32, 16384, 0))) != 0   # fixed at creation
    chid = lib.urpc_channel_create()
    assert chid >= 0 and lib.urpc_channel_queue_add(chid, ctypes.c_uint64(qh)) == 0
    assert lib.urpc_channel_queue_add(ch0.id, ctypes.c_uint64(qh)) != 0                 # ch0 is attached
    assert lib.urpc_channel_queue_pair(chid, ctypes.c_uint64(qh)) != 0                  # not attached yet
    assert lib.urpc_channel_server_attach(chid, srv.ip.encode(), srv.port) == 0
    assert lib.urpc_channel_queue_pair(chid, ctypes.c_uint64(qh)) == 0
    q = (ctypes.c_uint64 * 1)()
    assert lib.urpc_channel_queue_query(chid, q, 1) == 1 and q[0] == qh
    # a call through the explicit queue
    arg = ctypes.create_string_buffer(b"via my queue", 12)
    sge = urpc._Sge(ctypes.cast(arg, ctypes.c_void_p), 12)
    wr = urpc._CallWr(1, ctypes.pointer(sge), 1, 0)
    rsp, n = ctypes.create_string_buffer(64), ctypes.c_uint32(0)
    opt = urpc._CallOpt(0, 1, ctypes.cast(rsp, ctypes.c_void_p), 64, ctypes.pointer(n))
    assert lib.urpc_func_call(chid, ctypes.byref(wr), ctypes.byref(opt)) == 0 and rsp.raw[:n.value] == b"eueuq ym aiv"
    assert lib.urpc_queue_destroy(ctypes.c_uint64(qh)) != 0                             # still in use
    assert lib.urpc_channel_queue_unpair(chid, ctypes.c_uint64(qh)) == 0
    assert lib.urpc_channel_queue_rm(chid, ctypes.c_uint64(qh)) == 0
    assert lib.urpc_channel_destroy(chid) == 0
    assert lib.urpc_queue_destroy(ctypes.c_uint64(qh)) == 0
    # allocator plug-in
    lib.urpc_rsp_copy.restype = ctypes.c_void_p
    p = lib.urpc_rsp_copy(b"keep me", 7)
    assert ctypes.string_at(p, 7) == b"keep me"
    lib.urpc_rsp_free(ctypes.c_void_p(p))


@pytest.mark.parametrize("sealed", [False, True])
def test_several_queues_on_one_channel(tmp_path, sealed):
    """A channel with three explicit queues: all are paired during the attach, calls spread over them in turn or go to
    the queue the caller names, and each response returns on the queue of its request (clear and sealed)."""
    import ctypes
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    from umdk_b200 import urpc
    urpc.init(default_timeout_ms=2000)
    urpc.set_psk("5a" * 32 if sealed else "")
    srv = urpc.Server()
    srv.register(1, lambda b: b[::-1])
    lib = urpc._lib()
    lib.urpc_queue_create.restype = ctypes.c_uint64
    errors0 = urpc.stats()["errors"]                         # the counters outlive uninit
    try:
        qs = [lib.urpc_queue_create(None) for _ in range(3)]
        assert all(qs)
        chid = lib.urpc_channel_create()
        for q in qs:
            assert lib.urpc_channel_queue_add(chid, ctypes.c_uint64(q)) == 0
        assert lib.urpc_channel_queue_add(chid, ctypes.c_uint64(qs[1])) != 0          # already a lane of this channel
        other = lib.urpc_channel_create()
        assert lib.urpc_channel_queue_add(other, ctypes.c_uint64(qs[2])) != 0         # one queue serves one channel
        assert lib.urpc_channel_destroy(other) == 0
        got = (ctypes.c_uint64 * 4)()
        assert lib.urpc_channel_queue_query(chid, got, 4) == 3 and list(got)[:3] == qs
        assert lib.urpc_channel_server_attach(chid, srv.ip.encode(), srv.port) == 0
        for q in qs:
            assert lib.urpc_channel_queue_pair(chid, ctypes.c_uint64(q)) == 0

        def call(payload, on=None):
            arg = ctypes.create_string_buffer(payload, len(payload))
            sge = urpc._Sge(ctypes.cast(arg, ctypes.c_void_p), len(payload))
            wr = urpc._CallWr(1, ctypes.pointer(sge), 1, 0)
            rsp, n = ctypes.create_string_buffer(256), ctypes.c_uint32(0)
            opt = urpc._CallOpt(0, 1, ctypes.cast(rsp, ctypes.c_void_p), 256, ctypes.pointer(n))
            rc = (lib.urpc_func_call(chid, ctypes.byref(wr), ctypes.byref(opt)) if on is None else
                  lib.urpc_func_call_on(chid, ctypes.c_uint64(on), ctypes.byref(wr), ctypes.byref(opt)))
            return rc, rsp.raw[:n.value]

        def tx_rx(q):
            st = (ctypes.c_uint64 * 4)()
            assert lib.urpc_queue_stats_get(ctypes.c_uint64(q), st, 4) == 4
            return st[0], st[2]

        for i in range(9):                                   # in turn: three requests and responses per lane
            msg = b"lane message %d" % i
            assert call(msg) == (0, msg[::-1])
        assert [tx_rx(q) for q in qs] == [(3, 3)] * 3
        for i in range(4):                                   # a named lane takes them all
            assert call(b"only here", on=qs[2]) == (0, b"ereh ylno")
        assert [tx_rx(q) for q in qs] == [(3, 3), (3, 3), (7, 7)]
        assert urpc.stats()["errors"] == errors0             # nothing failed a seal or replay check on any lane
        assert call(b"x", on=0xdead)[0] != 0                 # not a queue of this channel
        # a lane leaves only while detached; the next one moves up
        assert lib.urpc_channel_queue_rm(chid, ctypes.c_uint64(qs[0])) != 0
        assert lib.urpc_channel_server_detach(chid) == 0
        assert lib.urpc_channel_queue_rm(chid, ctypes.c_uint64(qs[0])) == 0
        assert lib.urpc_channel_queue_query(chid, got, 4) == 2 and list(got)[:2] == qs[1:]
        assert lib.urpc_queue_destroy(ctypes.c_uint64(qs[0])) == 0
        assert lib.urpc_queue_destroy(ctypes.c_uint64(qs[1])) != 0                    # still held by the channel
        assert lib.urpc_channel_server_attach(chid, srv.ip.encode(), srv.port) == 0   # two lanes this time
        for i in range(4):
            assert call(b"again %d" % i) == (0, (b"again %d" % i)[::-1])
        assert lib.urpc_channel_destroy(chid) == 0
        for q in qs[1:]:
            assert lib.urpc_queue_destroy(ctypes.c_uint64(q)) == 0
    finally:
        srv.stop()
        urpc.set_psk("")
        urpc.uninit()


def test_channel_binding_with_lanes_and_deferred_reply(rpc):
    """`Channel(queues=3)`: asynchronous calls spread over the lanes; a request that the application answers later
    (urpc_func_return) still gets its response on the lane it came in on."""
    import ctypes
    urpc, srv, _ = rpc
    lib = urpc._lib()
    ch = urpc.Channel(srv.ip, srv.port, queues=3)
    try:
        assert len(ch.queues) == 3
        for i in range(6):
            ch.call_async(1, b"abc%d" % i, user_ctx=i)
        got, deadline = {}, time.monotonic() + 5
        while len(got) < 6 and time.monotonic() < deadline:
            for ev, ctx, status, data in ch.poll():
                got[ctx] = data
        assert got == {i: (b"abc%d" % i)[::-1] for i in range(6)}
        assert ch.queue_stats() == [(2, 2)] * 3
        assert ch.call(1, b"named", queue=1) == b"deman" and ch.queue_stats()[1] == (3, 3)
        # function 77 has no handler: the request surfaces in the server's poll and is answered by hand
        srv.paused = True
        time.sleep(0.05)
        ch.call_async(77, b"answer me later", user_ctx=900, queue=2)
        msgs, n, deadline = (urpc._PollMsg * 4)(), 0, time.monotonic() + 5
        while n == 0 and time.monotonic() < deadline:
            n = lib.urpc_server_poll(msgs, 4)
        assert n == 1 and msgs[0].func_id == 77 and ctypes.string_at(msgs[0].data, msgs[0].len) == b"answer me later"
        assert lib.urpc_func_return(ctypes.byref(msgs[0]), b"late", 4, 0) == 0
        lib.urpc_msg_release(ctypes.byref(msgs[0]))
        out, deadline = [], time.monotonic() + 5
        while not out and time.monotonic() < deadline:
            out = ch.poll()
        assert [(ctx, data) for _, ctx, _, data in out] == [(900, b"late")]
        assert ch.queue_stats() == [(2, 2), (3, 3), (3, 3)]
    finally:
        srv.paused = False
        ch.close()


def test_many_channels_outgrow_the_first_buffer_pool(rpc):
    """Every queue keeps a full receive ring posted, so a dozen queues need more blocks than the pool starts with: the
    pool grows instead of failing sends (UMQ mempool state reports the larger total)."""
    import ctypes
    urpc, srv, ch0 = rpc
    chans = [urpc.Channel(srv.ip, srv.port) for _ in range(6)]
    try:
        for i, ch in enumerate(chans):
            assert ch.call(1, b"channel %d" % i) == (b"channel %d" % i)[::-1]
        from umdk_b200 import umq

        class State(ctypes.Structure):
            _fields_ = [("block_size", ctypes.c_uint64), ("blocks_total", ctypes.c_uint64),
                        ("blocks_free", ctypes.c_uint64), ("generation", ctypes.c_uint64), ("registered", ctypes.c_int)]
        buf = ctypes.create_string_buffer(256)
        assert umq._lib().umq_mempool_state_get(ctypes.c_uint64(0), 0, buf) == 0
        st = State.from_buffer(buf)
        assert st.block_size == 65536 and st.blocks_total > 1024   # 64 MiB of 64 KiB blocks at the start
    finally:
        for ch in chans:
            ch.close()


def test_sealed_lane_with_four_threads_replying_at_once(tmp_path):
    """With a pre-shared key every message carries a counter that the receiver checks for replays. Four application
    threads answer deferred requests of ONE lane at the same time: counters must reach the wire in an order the
    receiver accepts, so every one of the replies arrives."""
    import ctypes
    import threading
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    from umdk_b200 import urpc
    urpc.set_psk("3a" * 32, "rpc")
    urpc.init(default_timeout_ms=5000)
    srv = urpc.Server()
    lib = urpc._lib()
    ch = None
    try:
        ch = urpc.Channel(srv.ip, srv.port)
        srv.paused = True
        time.sleep(0.05)
        N = 32
        for i in range(N):
            ch.call_async(77, b"req %02d" % i, user_ctx=i)
        msgs = (urpc._PollMsg * N)()
        n, deadline = 0, time.monotonic() + 5
        while n < N and time.monotonic() < deadline:
            got = lib.urpc_server_poll(ctypes.byref(msgs, n * ctypes.sizeof(urpc._PollMsg)), N - n)
            n += max(got, 0)
        assert n == N
        rcs = [None] * N

        def answer(lo, hi):
            for j in range(lo, hi):
                body = b"rsp " + ctypes.string_at(msgs[j].data, msgs[j].len)
                rcs[j] = lib.urpc_func_return(ctypes.byref(msgs[j]), body, len(body), 0)

        ths = [threading.Thread(target=answer, args=(k * 8, k * 8 + 8)) for k in range(4)]
        for t in ths:
            t.start()
        for t in ths:
            t.join()
        assert rcs == [0] * N
        for j in range(N):
            lib.urpc_msg_release(ctypes.byref(msgs[j]))
        out, deadline = {}, time.monotonic() + 5
        while len(out) < N and time.monotonic() < deadline:
            for _, ctx, status, data in ch.poll():
                assert status == 0
                out[ctx] = data
        assert out == {i: b"rsp req %02d" % i for i in range(N)}
    finally:
        srv.paused = False
        if ch is not None:
            ch.close()
        srv.stop()
        urpc.uninit()
        urpc.set_psk("", "")


def test_units_selftest():
    """Timer wheel, slab, id generator, head codecs and version negotiation, checked inside the library."""
    from umdk_b200 import _native
    assert _native.urpc().urpc_units_selftest() == 0


def _wait(cond, seconds=5.0):
    deadline = time.monotonic() + seconds
    while time.monotonic() < deadline:
        if cond():
            return True
        time.sleep(0.002)
    return cond()


def test_queues_join_and_leave_an_attached_channel(rpc):
    urpc, srv, ch = rpc
    assert ch.protocol() == (2, urpc.CAP_LIVE_QUEUES | urpc.CAP_ACK | urpc.CAP_TASK_CANCEL)
    assert ch.call(1, b"abc") == b"cba"
    before = urpc.ctl_stats()
    qa = ch.add_queue()            # control message QUEUE_ADD -> a new queue pair, usable at once
    qb = ch.add_queue()
    assert (qa, qb) == (0, 1)
    assert ch.call(1, b"on a", queue=qa) == b"a no" and ch.call(1, b"on b", queue=qb) == b"b no"
    for i in range(30):            # calls without a named queue take the lanes in turn
        assert ch.call(2, bytes([i])) == str(i).encode()
    sent = [s for s, _ in ch.queue_stats()]
    assert all(n >= 10 for n in sent), sent
    assert "lanes 3 live" in urpc.admin_query("sessions")
    # leave while calls are in flight on the lane: every one of them still gets its answer
    srv.paused = True
    for i in range(6):
        ch.call_async(1, bytes([97 + i]) * 4, user_ctx=i, queue=qa)
    srv.paused = False
    ch.remove_queue(qa)
    got = {}
    assert _wait(lambda: got.update({c: d for _, c, _, d in ch.poll()}) or len(got) == 6)
    assert got == {i: bytes([97 + i]) * 4 for i in range(6)}
    assert len(ch.queues) == 1 and ch.call(1, b"still b", queue=0) == b"b llits"
    assert "lanes 2 live" in urpc.admin_query("sessions")
    # a queue that joins later gets a new lane id (a sealing salt is never used twice)
    qc = ch.add_queue()
    assert ch.call(1, b"c", queue=qc) == b"c"
    after = urpc.ctl_stats()
    assert after["tasks_done"] - before["tasks_done"] == 4 and after["tasks_live"] == 0
    assert after["tasks_failed"] == before["tasks_failed"]
    assert "tasks_done" in urpc.admin_query("tasks")


def test_live_queue_changes_on_a_sealed_channel(tmp_path):
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    from umdk_b200 import urpc
    urpc.set_psk("3e" * 32, "rpc")
    urpc.init(default_timeout_ms=2000)
    srv = urpc.Server()
    try:
        srv.register(1, lambda b: b.upper())
        ch = urpc.Channel(srv.ip, srv.port)
        errors = urpc.stats()["errors"]
        q = ch.add_queue()
        for i in range(20):
            assert ch.call(1, b"sealed %d" % i, queue=q) == b"SEALED %d" % i
        ch.remove_queue(q)
        q2 = ch.add_queue()
        assert ch.call(1, b"again", queue=q2) == b"AGAIN"
        assert urpc.stats()["errors"] == errors     # nothing failed a seal check
        ch.close()
    finally:
        srv.stop()
        urpc.uninit()
        urpc.set_psk("", "")


def test_acknowledgement_cancel_and_function_notice(rpc):
    urpc, srv, ch = rpc
    srv.deferred = lambda fid, args: (b"late:" + args) if fid == 9 else None
    srv.defer_s = 0.15
    rid = ch.call_async(9, b"x", user_ctx=5, want_ack=True)
    events = []
    assert _wait(lambda: events.extend(ch.poll()) or len(events) >= 2)
    assert [(e[0], e[1]) for e in events] == [(urpc.POLL_ACK, 5), (urpc.POLL_RSP, 5)] and events[1][3] == b"late:x"
    # without want_ack there is no acknowledgement event
    ch.call_async(9, b"y", user_ctx=6)
    events = []
    assert _wait(lambda: events.extend(ch.poll()) or len(events) >= 1)
    time.sleep(0.05)
    events.extend(ch.poll())
    assert [(e[0], e[1]) for e in events] == [(urpc.POLL_RSP, 6)]
    # a cancelled call: the server drops its deferred answer instead of sending it
    srv.defer_s = 0.3
    n_ret = len(srv.return_codes)
    rid = ch.call_async(9, b"z", user_ctx=7)
    time.sleep(0.05)
    ch.cancel(rid)
    assert _wait(lambda: len(srv.return_codes) > n_ret)
    assert srv.return_codes[-1] == urpc.ERR_CANCELED
    time.sleep(0.05)
    assert ch.poll() == []
    srv.defer_s = 0.0
    # the server tells attached clients when its function table changes
    urpc.async_events()
    srv.register(33, lambda b: b)
    assert _wait(lambda: any(t == urpc.EVENT_FUNC_CHANGED and d == 1 for t, _, d in urpc.async_events()))
    assert ch.call(33, b"new") == b"new"


def test_detach_retires_the_session_on_the_server(rpc):
    urpc, srv, ch = rpc
    extra = urpc.Channel(srv.ip, srv.port, queues=2)
    assert extra.call(1, b"12") == b"21"
    before = urpc.ctl_stats()["sessions_retired"]
    extra.close()
    assert _wait(lambda: urpc.ctl_stats()["sessions_retired"] == before + 1)
    assert "retired" in urpc.admin_query("sessions")
    assert ch.call(1, b"ok") == b"ko"          # the other session is untouched


_PEER = r"""
import sys, time
from umdk_b200 import urpc
urpc.init(default_timeout_ms=2000)
srv = urpc.Server()
srv.register(1, lambda b: b[::-1])
print(srv.port, flush=True)
sys.stdin.readline()
srv.stop()
urpc.uninit()
"""


@pytest.mark.parametrize("server_max,client_env,want", [
    ("1", {}, (1, 0)),                                   # old server, new client: falls back to version 1
    (None, {"URPC_PROTO_MAX": "1"}, (1, 0)),             # new server, old client
    ("1", {"URPC_PROTO_MIN": "2"}, None),                # client insists on 2, server only has 1: refused
])
def test_version_negotiation_between_old_and_new_builds(tmp_path, server_max, client_env, want):
    import subprocess
    import sys
    shm = tmp_path / "urma"
    shm.mkdir(exist_ok=True)
    env = dict(os.environ, URMA_SHM_DIR=str(shm))
    if server_max:
        env["URPC_PROTO_MAX"] = server_max
    peer = subprocess.Popen([sys.executable, "-c", _PEER], env=env, stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                            text=True)
    os.environ["URMA_SHM_DIR"] = str(shm)
    from umdk_b200 import urpc
    try:
        port = int(peer.stdout.readline())
        os.environ.update(client_env)
        urpc.init(default_timeout_ms=2000)
        if want is None:
            with pytest.raises(urpc.UrpcError) as e:
                urpc.Channel("127.0.0.1", port)
            assert e.value.code == urpc.ERR_VERSION
        else:
            ch = urpc.Channel("127.0.0.1", port)
            assert ch.protocol() == want
            assert ch.call(1, b"compat") == b"tapmoc"
            rid = ch.call_async(1, b"q", user_ctx=3, want_ack=True)   # no acknowledgements in version 1
            got = []
            assert _wait(lambda: got.extend(ch.poll()) or got)
            assert [(g[0], g[1]) for g in got] == [(urpc.POLL_RSP, 3)]
            with pytest.raises(urpc.UrpcError):
                ch.add_queue()                         # queues change only while detached with such a peer
            ch.close()
    finally:
        for k in client_env:
            os.environ.pop(k, None)
        urpc.uninit()
        peer.stdin.write("\n")
        peer.stdin.flush()
        peer.wait(timeout=20)


def test_server_threads_serve_their_own_share_of_the_clients(tmp_path):
    """Two polling threads on the server: each serves the sessions whose number is its own modulo two, so with four
    attached channels both threads get requests and every call is answered exactly once."""
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    from umdk_b200 import urpc
    urpc.init(default_timeout_ms=3000)
    srv = urpc.Server(threads=2)
    srv.register(1, lambda b: b[::-1])                       # runs inside the library on whichever thread polls
    srv.deferred = lambda fid, args: b"d:" + args            # function 5 has no handler: handed to the thread
    chans = [urpc.Channel(srv.ip, srv.port) for _ in range(4)]
    try:
        for rnd in range(20):
            for i, ch in enumerate(chans):
                assert ch.call(1, b"abc%d" % i) == (b"abc%d" % i)[::-1]
                assert ch.call(5, b"x%d.%d" % (i, rnd)) == b"d:x%d.%d" % (i, rnd)
        assert sum(srv.served_by) == 80 and min(srv.served_by) > 0, srv.served_by
        assert urpc._lib().urpc_server_poll_shard(2, 2, None, 0) < 0     # shard out of range
    finally:
        for ch in chans:
            ch.close()
        srv.stop()
        urpc.uninit()
