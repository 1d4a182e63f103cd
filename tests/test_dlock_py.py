"""Distributed locks through the Python binding: two clients contend for exclusive, shared and fair locks with
leases, and hammer a shared 64-bit object with fetch-add / compare-and-swap from threads."""
import os
import threading
import time

import pytest


@pytest.fixture()
def service(tmp_path):
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    from umdk_b200 import dlock
    srv = dlock.Server()
    a, b = dlock.Client(srv.ip, srv.port), dlock.Client(srv.ip, srv.port)
    yield dlock, srv, a, b
    a.close()
    b.close()
    srv.stop()


def test_exclusive_shared_and_lease(service):
    dlock, srv, a, b = service
    la, lb = a.get_lock("L1", dlock.ATOMIC), b.get_lock("L1", dlock.ATOMIC)
    assert a.trylock(la) is True
    assert b.trylock(lb) is False                 # held by a
    with pytest.raises(dlock.DlockError):
        b.unlock(lb)                              # not the owner
    a.unlock(la)
    assert b.trylock(lb) is True
    b.unlock(lb)
    # readers share, a writer waits for them
    ra, rb = a.get_lock("RW1", dlock.RW), b.get_lock("RW1", dlock.RW)
    assert a.trylock(ra, shared=True) and b.trylock(rb, shared=True)
    a.unlock(ra)
    b.unlock(rb)
    assert b.trylock(rb) is True
    b.unlock(rb)
    # a lease that runs out can be taken over
    assert a.trylock(la, expire_ms=100) is True
    time.sleep(0.3)
    assert b.trylock(lb, expire_ms=1000) is True
    b.unlock(lb)
    assert srv.stats()["expired_takeover"] >= 1


def test_fair_lock_blocks_until_released(service):
    dlock, srv, a, b = service
    fa, fb = a.get_lock("F1", dlock.FAIR), b.get_lock("F1", dlock.FAIR)
    a.lock(fa)
    got = []

    def waiter():
        b.lock(fb, timeout_ms=5000)
        got.append(time.monotonic())
        b.unlock(fb)

    t = threading.Thread(target=waiter)
    t.start()
    time.sleep(0.2)
    released = time.monotonic()
    a.unlock(fa)
    t.join(timeout=10)
    assert got and got[0] >= released


def test_atomic_object_from_two_clients(service):
    dlock, srv, a, b = service
    oa = a.atomic_create("counter", 5)
    ob = b.atomic_get("counter")

    def hammer(cl, oid):
        for _ in range(2000):
            cl.atomic_faa(oid, 1)

    ts = [threading.Thread(target=hammer, args=(a, oa)), threading.Thread(target=hammer, args=(b, ob))]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert a.atomic_snapshot(oa) == 5 + 4000
    assert b.atomic_cas(ob, 4005, 1) == 4005 and a.atomic_snapshot(oa) == 1
    assert b.atomic_cas(ob, 4005, 2) == 1 and a.atomic_snapshot(oa) == 1


def test_secured_service_locks_work_and_wrong_keys_are_refused(tmp_path):
    """With a pre-shared key the control channel is TLS 1.3 PSK and lock commands are sealed; a client with another
    key or with none cannot join, and the server counts the refusals."""
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    from umdk_b200 import dlock
    key = "a1" * 32
    dlock.set_psk(key, "locks")
    srv = None
    try:
        srv = dlock.Server()
        a, b = dlock.Client(srv.ip, srv.port), dlock.Client(srv.ip, srv.port)
        la, lb = a.get_lock("S1", dlock.ATOMIC), b.get_lock("S1", dlock.ATOMIC)
        assert a.trylock(la) is True and b.trylock(lb) is False
        a.unlock(la)
        assert b.trylock(lb) is True
        b.unlock(lb)
        obj = a.atomic_create("ctr", 5)
        assert a.atomic_faa(obj, 3) == 5 and b.atomic_snapshot(b.atomic_get("ctr")) == 8
        assert a.heartbeat() == 0
        st = srv.stats()
        assert st["sealed_rejected"] == 0 and st["tls_rejected"] == 0 and st["data_msgs"] >= 4
        for bad_key, ident in (("b2" * 32, "locks"), (key, "other"), ("", "")):
            dlock.set_psk(bad_key, ident)
            with pytest.raises(dlock.DlockError):
                dlock.Client(srv.ip, srv.port)
        assert srv.stats()["tls_rejected"] == 3
        dlock.set_psk(key, "locks")
        a.close()
        b.close()
        with pytest.raises(dlock.DlockError):
            dlock.set_psk("zz", "")          # malformed keys are refused, never ignored
    finally:
        if srv is not None:
            srv.stop()
        dlock.set_psk("", "")


def test_async_request_batches_and_stat_reset(service):
    dlock, srv, a, b = service
    ids = [a.get_lock(f"B{i}", dlock.ATOMIC) for i in range(3)]
    # asynchronous lock: send, look, collect; a second request while one is outstanding is refused
    a.request_async(ids[0], dlock.EXCLUSIVE, expire_ms=2000)
    with pytest.raises(dlock.DlockError) as e:
        a.request_async(ids[1])
    assert e.value.code == dlock.EASYNC
    deadline = time.monotonic() + 3
    res = None
    while res is None and time.monotonic() < deadline:
        res = a.result()
    assert res == dlock.SUCCESS
    with pytest.raises(dlock.DlockError) as e:
        a.result()
    assert e.value.code == dlock.NO_ASYNC
    lb = b.get_lock("B0", dlock.ATOMIC)
    assert b.trylock(lb) is False                          # the asynchronous request really took the lock
    assert a.trylock(ids[1]) and a.trylock(ids[2])
    assert a.batch_extend(ids, 5000) == [0, 0, 0]
    assert a.batch_unlock(ids) == [0, 0, 0]
    assert b.trylock(lb) is True
    b.unlock(lb)
    assert a.batch_release(ids) == 0
    assert srv.stats()["trylock_ok"] >= 3
    srv.clear_stats()
    a.clear_stats()
    assert srv.stats()["trylock_ok"] == 0 and srv.stats()["clients"] == 2 and a.stats()["trylock_ok"] == 0
    a.reinit_done()                                        # harmless outside a recovery
