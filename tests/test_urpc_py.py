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

    class ChCfg(ctypes.Structure):
        _fields_ = [("timeout_ms", ctypes.c_uint32), ("attached", ctypes.c_int), ("lost", ctypes.c_int),
                    ("sealed", ctypes.c_int), ("pending_calls", ctypes.c_uint32), ("server_ip", ctypes.c_char * 64),
                    ("server_port", ctypes.c_uint16)]
    cfg = ChCfg()
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
