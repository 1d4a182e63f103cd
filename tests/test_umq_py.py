"""UMQ through the Python binding: two queues in one process bound to each other, ordered delivery of messages of
several sizes in both directions, more messages than the queue depth (credits must flow back), statistics."""
import os

import pytest


@pytest.fixture()
def pair(tmp_path):
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    from umdk_b200 import umq
    umq.init(flow_control=True)
    a, b = umq.Queue("a", depth=16), umq.Queue("b", depth=16)
    a.bind(b.bind_info())
    b.bind(a.bind_info())
    yield umq, a, b
    a.close()
    b.close()
    umq.uninit()


def test_messages_both_ways_in_order(pair):
    umq, a, b = pair
    msgs = [bytes([i % 251]) * (1 + 37 * i) for i in range(100)]   # up to ~3.7 KB, more than the depth of 16
    for i, m in enumerate(msgs):
        a.send(m)
        if i % 4 == 3:                       # the receiver drains as we go, returning credits
            for j in range(i - 3, i + 1):
                assert b.recv() == msgs[j]
    b.send(b"pong" * 100)
    assert a.recv() == b"pong" * 100
    assert a.recv(timeout_s=0.05) is None
    st = a.io_stats()
    assert st["tx_msgs"] >= 100 and st["tx_bytes"] >= sum(map(len, msgs))
    assert b.flow_control_stats()["credits_returned"] > 0 or b.flow_control_stats()["credits_granted"] > 0


def test_trace_records_every_operation(pair, tmp_path):
    umq, a, b = pair
    path = tmp_path / "umq.trace"
    umq.trace_start(str(path), flush_interval_ms=20)
    for i in range(40):
        a.send(bytes([i]) * 100)
        assert b.recv() == bytes([i]) * 100
    import time
    time.sleep(0.1)                       # let the timer flush at least once while the trace is running
    mid = path.read_text().count("\n")
    st = umq.trace_stop()
    lines = [l.split() for l in path.read_text().splitlines() if not l.startswith("#")]
    assert mid > 1 and st["dropped"] == 0 and st["written"] == len(lines)
    kinds = {l[2] for l in lines}
    assert {"enqueue", "dequeue", "buf_alloc"} <= kinds
    assert sum(1 for l in lines if l[2] == "enqueue") >= 40
    assert all(int(l[0]) > 0 and int(l[3]) >= 0 for l in lines)
    # a second trace with a tiny ring overflows between flushes: entries are dropped and counted, nothing blocks
    umq.trace_start(str(tmp_path / "t2.trace"), flush_interval_ms=2000, ring_entries=8)
    for i in range(40):
        a.send(b"x")
        assert b.recv() == b"x"
    st2 = umq.trace_stop()
    assert st2["dropped"] > 0 and st2["written"] <= 8 * 4


def test_perf_callback_log_sink_and_error_event(pair):
    umq, a, b = pair
    seen, logs = [], []
    umq.io_perf_callback(lambda rec, ns: seen.append((rec, ns)))
    umq.log_config(3, lambda lvl, msg: logs.append((lvl, msg)))
    try:
        a.send(b"hello")
        assert b.recv() == b"hello"
        assert {"enqueue", "dequeue", "buf_alloc"} <= {r for r, _ in seen} and all(ns >= 0 for _, ns in seen)
        assert umq.async_events() == []
        a.set_state(2)
        ev = umq.async_events()
        assert ev == [(1, a.h, 0)] and a.state() == 2
        assert any("state" in m for _, m in logs)
        a.set_state(1)
    finally:
        umq.io_perf_callback(None)
        umq.log_config(1, None)
