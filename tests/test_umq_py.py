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
