"""Host-side membership view: ranks learn of an orderly departure and of a silent rank before their next step.
CPU ranks only (gloo-style processes sharing a TCP store); no device is involved."""
import socket
import time

import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    try:
        from umdk_b200.parallel.membership import Membership
        store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=30))
        m = Membership(store, rank, world, timeout_s=0.6)
        assert m.wait_for_all(20)
        steps = []
        for step in range(40):
            m.beat()
            alive = m.alive()
            steps.append(sorted(alive))
            if rank == 1 and step == 3:
                m.leave()                       # orderly: tells the others, then goes
                break
            if rank == 2 and step == 6:
                break                           # dies silently: no leave(), heartbeats just stop
            if alive == {0}:
                break                           # rank 0 is alone: nothing left to coordinate
            time.sleep(0.1)
        q.put((rank, steps))
        if rank == 0:
            time.sleep(0.5)                     # keep the store up until the others have reported
    except Exception:
        import traceback
        q.put((rank, "ERR " + traceback.format_exc()))


def test_departure_and_silence_are_seen_before_the_next_step():
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=60) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
    for r, v in got.items():
        assert not isinstance(v, str), v
    views = got[0]
    assert views[0] == [0, 1, 2]
    first_without_1 = next(i for i, v in enumerate(views) if 1 not in v)
    first_without_2 = next(i for i, v in enumerate(views) if 2 not in v)
    assert 3 <= first_without_1 <= 6             # rank 1 announced at its step 3
    assert first_without_2 > first_without_1     # rank 2 went silent later and is dropped after the timeout
    assert views[-1] == [0]
