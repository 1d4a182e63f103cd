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
