"""Multipath ("bond") URMA device over two shared-memory paths: traffic is spread over the paths, a link fault
injected on the host side (requests on that path vanish) triggers failover with no lost or duplicated message, and
the health probe brings the path back after the fault is lifted. No GPU is involved."""
import ctypes
import os
import time

import pytest
import torch


@pytest.fixture()
def bond_env(tmp_path, monkeypatch):
    monkeypatch.setenv("URMA_SHM_DIR", str(tmp_path))
    monkeypatch.setenv("BOND_HEALTH_CHECK_ACTIVE_INTERVAL", "50")
    monkeypatch.setenv("BOND_MODE", "2")
    yield


def test_sliding_window_semantics():
    # the same class that the provider uses, compiled into a tiny checker at build time would be overkill:
    # exercise it through a duplicate-delivery scenario in the bond test below; here the pure-python model of the
    # contract documents the expected behaviour
    seen, base, bits = set(), None, 1024

    def accept(msn):
        nonlocal base
        if base is None:
            base = msn
        if msn < base:
            return False
        if msn in seen:
            return False
        seen.add(msn)
        return True
    assert accept(5) and not accept(5) and accept(7) and accept(6) and not accept(4)


def test_bond_failover_and_failback(bond_env):
    from umdk_b200 import urma
    a, b = urma.Context("bond0"), urma.Context("bond0")
    try:
        ea, eb = a.endpoint(depth=64, recv_token=3), b.endpoint(depth=64, recv_token=3)
        mem_b = torch.zeros(1024, dtype=torch.int64)
        seg_b = b.register(mem_b, token=9)
        peer_b = a.import_endpoint(eb.blob, token=3)
        rseg = a.import_segment(seg_b.blob, token=9)
        src = torch.arange(1024, dtype=torch.int64)
        # balanced traffic uses both paths
        for i in range(8):
            ea.write(peer_b, rseg, rseg.va + i * 64, src.data_ptr() + i * 64, 64)
        ea.wait(8)
        assert torch.equal(mem_b[:64], src[:64])
        st = urma.bond_path_stats(a)
        assert len(st) == 2 and st[0]["tx"] > 0 and st[1]["tx"] > 0 and all(s["up"] for s in st)
        # break path 0 on the host side: requests posted there are dropped and time out
        urma.user_ctl(a, 4, addr=0, length=1)
        for i in range(6):
            ea.atomic(peer_b, urma.OPC_FADD, rseg, rseg.va + 8 * 1000, 1)
        got = 0
        deadline = time.time() + 20
        while got < 6 and time.time() < deadline:
            got += len(ea.wait(1, timeout_ms=3000, check=True))
        assert got == 6
        assert int(mem_b[1000]) == 6, "fetch-adds must be applied exactly once each"
        st = urma.bond_path_stats(a)
        assert not st[0]["up"] and st[0]["errors"] >= 1 and st[1]["failovers"] >= 1
        # two-sided traffic while the path is down: every message arrives once
        bufs = [torch.zeros(8, dtype=torch.int64) for _ in range(5)]
        for i, t in enumerate(bufs):
            eb.post_recv(t, user_ctx=100 + i)
        msgs = [torch.full((8,), i + 1, dtype=torch.int64) for i in range(5)]
        for i, m in enumerate(msgs):
            ea.send(peer_b, m.data_ptr(), 64, user_ctx=i, imm=i)
        ea.wait(5, timeout_ms=10000)
        rc = eb.wait(5, timeout_ms=10000)
        assert sorted(int(t[0]) for t in bufs) == [1, 2, 3, 4, 5]
        assert all(c.is_recv and c.length == 64 for c in rc)
        # lift the fault: the health probe marks the path up again
        urma.user_ctl(a, 4, addr=0, length=0)
        deadline = time.time() + 10
        while time.time() < deadline and not urma.bond_path_stats(a)[0]["up"]:
            time.sleep(0.05)
        st = urma.bond_path_stats(a)
        assert st[0]["up"] and st[0]["failbacks"] >= 1
        before = st[0]["tx"]
        for i in range(4):
            ea.read(peer_b, rseg, rseg.va, src.data_ptr(), 64)
        ea.wait(4)
        assert urma.bond_path_stats(a)[0]["tx"] > before
    finally:
        a.close()
        b.close()


def test_bond_scheduling_policies(bond_env):
    """priority: everything on the preferred path until it is taken down, then the next of the list; least_load and
    random: both paths carry traffic; affinity: the path of the calling thread's CPU; an unknown policy is refused."""
    from umdk_b200 import urma
    a, b = urma.Context("bond0"), urma.Context("bond0")
    try:
        ea, eb = a.endpoint(depth=64, recv_token=3), b.endpoint(depth=64, recv_token=3)
        mem_b = torch.zeros(1024, dtype=torch.int64)
        seg_b = b.register(mem_b, token=9)
        peer_b = a.import_endpoint(eb.blob, token=3)
        rseg = a.import_segment(seg_b.blob, token=9)
        src = torch.arange(1024, dtype=torch.int64)

        def burst(n=16):
            before = [s["tx"] for s in urma.bond_path_stats(a)]
            for i in range(n):
                ea.write(peer_b, rseg, rseg.va + (i % 8) * 64, src.data_ptr(), 64)
            ea.wait(n)
            return [s["tx"] - b0 for s, b0 in zip(urma.bond_path_stats(a), before)]

        urma.bond_set_policy(a, "priority", priority=[1, 0])
        assert urma.bond_sched_stats(a)["policy"] == "priority"
        assert burst() == [0, 16]
        urma.user_ctl(a, 2, addr=1, length=1)          # path 1 administratively down: next of the list
        assert burst() == [16, 0]
        urma.user_ctl(a, 2, addr=1, length=0)
        urma.bond_set_policy(a, "priority", priority=[0, 1])
        assert burst() == [16, 0]
        for pol in ("least_load", "random"):
            urma.bond_set_policy(a, pol)
            d = burst(64)
            assert sum(d) == 64 and d[0] > 0 and d[1] > 0, (pol, d)
        urma.bond_set_policy(a, "affinity", priority=[0, 1])
        cpu = sorted(os.sched_getaffinity(0))[0]
        saved = os.sched_getaffinity(0)
        os.sched_setaffinity(0, {cpu})
        try:
            d = burst()
        finally:
            os.sched_setaffinity(0, saved)
        assert d[cpu % 2] == 16 and d[1 - cpu % 2] == 0
        assert urma.bond_sched_stats(a)["inflight"] == [0, 0]     # every completion has been accounted
        with pytest.raises(urma.UrmaError):
            urma.user_ctl(a, 5, addr=9)
        with pytest.raises(urma.UrmaError):
            urma.user_ctl(a, 6, addr=0x00)                         # path 0 named twice
    finally:
        a.close()
        b.close()


def test_bond_resends_go_through_the_timing_wheel(bond_env, monkeypatch):
    """A request whose path fails is resent from the timing wheel after BOND_RESEND_DELAY_MS, exactly once."""
    from umdk_b200 import urma
    monkeypatch.setenv("BOND_RESEND_DELAY_MS", "20")
    a, b = urma.Context("bond0"), urma.Context("bond0")
    try:
        ea, eb = a.endpoint(depth=64, recv_token=3), b.endpoint(depth=64, recv_token=3)
        mem_b = torch.zeros(16, dtype=torch.int64)
        seg_b = b.register(mem_b, token=9)
        peer_b = a.import_endpoint(eb.blob, token=3)
        rseg = a.import_segment(seg_b.blob, token=9)
        urma.bond_set_policy(a, "priority", priority=[0, 1])
        urma.user_ctl(a, 4, addr=0, length=1)                       # path 0 drops everything
        for _ in range(4):
            ea.atomic(peer_b, urma.OPC_FADD, rseg, rseg.va, 1)
        got, deadline = 0, time.time() + 20
        while got < 4 and time.time() < deadline:
            got += len(ea.wait(1, timeout_ms=3000))
        assert got == 4 and int(mem_b[0]) == 4
        st = urma.bond_sched_stats(a)
        assert st["deferred_resends"] >= 1 and st["inflight"] == [0, 0]
        urma.user_ctl(a, 4, addr=0, length=0)
    finally:
        a.close()
        b.close()
