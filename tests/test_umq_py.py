"""UMQ through the Python binding: two queues in one process bound to each other, ordered delivery of messages of
several sizes in both directions, more messages than the queue depth (credits must flow back), statistics."""
import ctypes
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


def test_buffer_lists_queries_and_transport_pool(pair):
    """The helper calls around the queue: list surgery on buffers, configuration / device / pool queries, user
    control, text forms of the statistics, and a transport pool that watches several queues through one eventfd."""
    import ctypes
    umq, a, b = pair
    lib = umq._lib()
    Buf = umq._Buf
    lib.umq_buf_alloc.restype = ctypes.POINTER(Buf)
    lib.umq_buf_break_and_free.restype = ctypes.POINTER(Buf)
    lib.umq_data_to_head.restype = ctypes.POINTER(Buf)
    lib.umq_data_to_head.argtypes = [ctypes.c_void_p]
    # three buffers of 100 bytes in one list; cut after the first
    head = lib.umq_buf_alloc(100, 3, ctypes.c_uint64(a.h))
    assert head and head.contents.total_data_size == 300
    second = ctypes.cast(head.contents.qbuf_next, ctypes.POINTER(Buf))   # a copy of the pointer, not a view
    assert lib.umq_buf_split(head, second) == 0
    assert head.contents.total_data_size == 100 and not head.contents.qbuf_next
    assert second.contents.total_data_size == 200
    assert lib.umq_buf_split(head, second) != 0                      # no longer on that list
    # a pointer into a data area leads back to its buffer
    inner = ctypes.c_void_p(second.contents.buf_data + 17)
    back = lib.umq_data_to_head(inner)
    assert ctypes.addressof(back.contents) == ctypes.addressof(second.contents)
    assert not lib.umq_data_to_head(ctypes.c_void_p(ctypes.addressof(ctypes.c_int(0))))
    # two messages back to back: the first is freed, the second returned
    second.contents.total_data_size = 100                             # message 1 = one buffer, message 2 = the next
    third = ctypes.cast(second.contents.qbuf_next, ctypes.POINTER(Buf))
    third.contents.total_data_size = 100
    rest = lib.umq_buf_break_and_free(second)
    assert ctypes.addressof(rest.contents) == ctypes.addressof(third.contents)
    lib.umq_buf_free(rest)
    lib.umq_buf_free(head)

    class CfgGet(ctypes.Structure):
        _fields_ = [("create_option", umq._CreateOpt), ("state", ctypes.c_int), ("feature", ctypes.c_uint32),
                    ("trans_mode", ctypes.c_int), ("block_size", ctypes.c_uint32)]
    cfg = CfgGet()
    assert lib.umq_cfg_get(ctypes.c_uint64(a.h), ctypes.byref(cfg)) == 0
    assert cfg.create_option.name == b"a" and cfg.state == 1 and cfg.block_size >= 8192

    class DevInfo(ctypes.Structure):
        _fields_ = [("dev_name", ctypes.c_char * 64), ("eid", ctypes.c_uint8 * 16), ("trans_mode", ctypes.c_int),
                    ("max_msg_size", ctypes.c_uint64), ("port_cnt", ctypes.c_uint32)]
    n = ctypes.c_int(0)
    lib.umq_dev_info_list_get.restype = ctypes.POINTER(DevInfo)
    devs = lib.umq_dev_info_list_get(0, ctypes.byref(n))
    names = {devs[i].dev_name for i in range(n.value)}
    assert {b"shm0", b"shm1"} <= names
    lib.umq_dev_info_list_free(0, devs)
    assert lib.umq_dev_add(b"shm1") == 0 and lib.umq_dev_add(b"nope") != 0

    class Pool(ctypes.Structure):
        _fields_ = [(k, ctypes.c_uint64) for k in ("block_size", "blocks_total", "blocks_free", "generation")] + \
                   [("registered", ctypes.c_int)]
    st = Pool()
    assert lib.umq_mempool_state_get(ctypes.c_uint64(a.h), 0, ctypes.byref(st)) == 0 and st.registered == 1
    gen = st.generation
    assert lib.umq_mempool_state_refresh(ctypes.c_uint64(a.h), 0) == 0
    lib.umq_mempool_state_get(ctypes.c_uint64(a.h), 0, ctypes.byref(st))
    assert st.generation == gen + 1 and lib.umq_mempool_state_get(ctypes.c_uint64(a.h), 7, ctypes.byref(st)) != 0

    # transport pool over both queues: nothing ready, then a message for b
    lib.umq_transport_pool_resource_create.restype = ctypes.c_uint64
    pool = lib.umq_transport_pool_resource_create()
    assert pool and lib.umq_transport_pool_eventfd_get(ctypes.c_uint64(pool)) >= 0
    for q in (a, b):
        assert lib.umq_transport_pool_resource_modify(ctypes.c_uint64(pool), ctypes.c_uint64(q.h), 1) == 0
    assert lib.umq_transport_pool_resource_modify(ctypes.c_uint64(pool), ctypes.c_uint64(a.h), 1) != 0   # twice

    class PoolStats(ctypes.Structure):
        _fields_ = [("queues", ctypes.c_uint32), ("queues_ready", ctypes.c_uint32), ("wakeups", ctypes.c_uint64)]
    ps = PoolStats()
    assert lib.umq_stats_transport_pool_get(ctypes.c_uint64(pool), ctypes.byref(ps)) == 0
    assert (ps.queues, ps.queues_ready) == (2, 0)
    a.send(b"wake up")
    import time
    deadline = time.monotonic() + 2
    while ps.queues_ready == 0 and time.monotonic() < deadline:
        lib.umq_stats_transport_pool_get(ctypes.c_uint64(pool), ctypes.byref(ps))
    assert ps.queues_ready == 1 and ps.wakeups >= 1
    assert b.recv() == b"wake up"
    txt = ctypes.create_string_buffer(256)
    assert lib.umq_transport_pool_stats_to_str(ctypes.byref(ps), txt, 256) > 0 and b"queues 2" in txt.value
    assert lib.umq_transport_pool_resource_destroy(ctypes.c_uint64(pool)) == 0

    # user control, statistics as text, reset
    class CtlIn(ctypes.Structure):
        _fields_ = [("opcode", ctypes.c_uint32), ("arg", ctypes.c_uint64)]
    class CtlOut(ctypes.Structure):
        _fields_ = [("value", ctypes.c_uint64)]
    out = CtlOut()
    assert lib.umq_user_ctl(ctypes.c_uint64(b.h), ctypes.byref(CtlIn(1, 0)), ctypes.byref(out)) == 0
    assert lib.umq_user_ctl(ctypes.c_uint64(b.h), ctypes.byref(CtlIn(99, 0)), ctypes.byref(out)) != 0
    io = umq._IoStats()
    lib.umq_stats_io_get(ctypes.c_uint64(a.h), ctypes.byref(io))
    assert lib.umq_io_stats_to_str(ctypes.byref(io), txt, 256) > 0 and b"tx 1 msgs" in txt.value
    assert lib.umq_stats_io_reset(ctypes.c_uint64(a.h)) == 0 and a.io_stats()["tx_msgs"] == 0
    lvl = ctypes.c_int(-1)
    assert lib.umq_log_config_get(ctypes.byref(lvl)) == 0 and 0 <= lvl.value <= 4
    big = ctypes.create_string_buffer(2048)
    assert lib.umq_stats_perf_to_str(big, 2048) > 0 and b"enqueue" in big.value


def test_tiny_messages_come_from_the_tiny_pool(tmp_path):
    """Buffers of at most 512 bytes are served from the tiny pool (pool id 1) and leave the block pool untouched;
    a message sent from a tiny buffer arrives intact."""
    import ctypes
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    from umdk_b200 import umq
    lib = umq._lib()

    class State(ctypes.Structure):
        _fields_ = [("block_size", ctypes.c_uint64), ("blocks_total", ctypes.c_uint64),
                    ("blocks_free", ctypes.c_uint64), ("generation", ctypes.c_uint64), ("registered", ctypes.c_int)]

    def state(pool):
        st = State()
        assert lib.umq_mempool_state_get(ctypes.c_uint64(0), pool, ctypes.byref(st)) == 0
        return st

    umq.init()
    try:
        a, b = umq.Queue("tiny_a", depth=16), umq.Queue("tiny_b", depth=16)
        a.bind(b.bind_info())
        b.bind(a.bind_info())
        big0 = state(0).blocks_free
        bufs = [lib.umq_buf_alloc(100, 1, a.h) for _ in range(300)]
        assert all(bufs)
        t = state(1)
        assert t.block_size == 512 and t.blocks_total >= 1024 and t.registered == 1
        assert state(0).blocks_free >= big0 - 8          # the block pool did not pay for them
        for p in bufs:
            lib.umq_buf_free(p)
        a.send(b"tiny payload")
        assert b.recv() == b"tiny payload"
        assert lib.umq_mempool_state_get(ctypes.c_uint64(0), 2, ctypes.byref(State())) != 0
        a.close()
        b.close()
    finally:
        umq.uninit()


def test_transport_table_serves_queues_by_mode(pair):
    """Queues created with the in-process transport mode exchange buffers without touching URMA, side by side with
    queues on the URMA transport; a full receiver pushes back; a mode can be given a user-supplied table entry."""
    import ctypes
    umq, a, b = pair
    lib = umq._lib()
    lib.umq_transport_name.restype = ctypes.c_char_p
    assert lib.umq_transport_name(umq.TRANS_MODE_UB) == b"urma"
    assert lib.umq_transport_name(umq.TRANS_MODE_IPC) == b"ipc-local"
    x, y = umq.Queue("lx", depth=4, transport=umq.TRANS_MODE_IPC), umq.Queue("ly", depth=4, transport=umq.TRANS_MODE_IPC)
    try:
        x.bind(y.bind_info())
        y.bind(x.bind_info())
        for i in range(4):
            x.send(bytes([i]) * 1000)
        with pytest.raises(umq.UmqError):           # the receiver's ring of 4 is full
            x.send(b"one too many")
        assert [y.recv() for _ in range(4)] == [bytes([i]) * 1000 for i in range(4)]
        y.send(b"back")
        assert x.recv() == b"back" and x.recv(timeout_s=0.02) is None
        assert x.io_stats()["tx_msgs"] == 4 and y.io_stats()["rx_msgs"] == 4
        a.send(b"urma path still works")             # the URMA-backed pair is unaffected
        assert b.recv() == b"urma path still works"
        with pytest.raises(umq.UmqError):            # an in-process queue cannot bind to a URMA queue's blob
            x2 = umq.Queue("lz", transport=umq.TRANS_MODE_IPC)
            try:
                x2.bind(a.bind_info())
            finally:
                x2.close()
        assert lib.umq_transport_register(99, None) != 0
    finally:
        x.close()
        y.close()


def test_large_messages_are_pulled_by_the_receiver_and_keep_their_place(pair):
    """A message that does not fit the peer's receive buffers (8 KB blocks here) travels as a descriptor and the
    receiver reads it from the sender's memory; delivery order and flow control are the same as for small ones."""
    umq, a, b = pair
    big = [bytes([i + 1]) * (100_000 + 4321 * i) for i in range(4)] + [os.urandom(3 << 20)]
    order = []
    for i, m in enumerate(big):
        a.send(b"before %d" % i)
        a.send(m)
        a.send(b"after %d" % i)
        order += [b"before %d" % i, m, b"after %d" % i]
    for want in order:
        got = b.recv()
        assert got == want, (len(got or b""), len(want))
    assert b.recv(timeout_s=0.05) is None
    sa, sb = a.io_stats(), b.io_stats()
    assert sa["pull_tx"] == len(big) and sb["pull_rx"] == len(big) and sa["pull_rx"] == 0
    assert sa["tx_msgs"] == len(order) and sb["rx_msgs"] == len(order)
    assert sb["rx_bytes"] == sum(map(len, order)) and sa["tx_errors"] == 0 and sb["rx_errors"] == 0
    # more large messages than the queue depth, both directions at once: credits and buffers come back
    for i in range(40):
        a.send(bytes([i]) * 20_000)
        b.send(bytes([255 - i]) * 30_000)
        assert b.recv() == bytes([i]) * 20_000
        assert a.recv() == bytes([255 - i]) * 30_000
    pool = umq.qbuf_stats() if hasattr(umq, "qbuf_stats") else None
    if pool:
        assert pool["alloc_failures"] == 0


def test_sub_queues_share_receive_buffers_and_borrow_jetties(tmp_path):
    """Many sub queues on two main queues: no endpoint and no receive buffers of their own. Every pair keeps its
    own order and flow control, large messages are pulled, the jetty pool counts the borrowed posts."""
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    from umdk_b200 import umq
    umq.init(flow_control=True)
    made = []
    try:
        before = umq.jetty_pool_stats()
        ma = umq.Queue("main-a", depth=64, main=True, share_transport=True)
        mb = umq.Queue("main-b", depth=64, main=True, share_transport=True)
        made += [ma, mb]
        ma.bind(mb.bind_info())
        mb.bind(ma.bind_info())
        n_sub = 24
        sa = [umq.Queue(f"sa{i}", depth=8, sub_of=ma) for i in range(n_sub)]
        sb = [umq.Queue(f"sb{i}", depth=8, sub_of=mb) for i in range(n_sub)]
        made = sa + sb + made          # closed in this order: sub queues first
        for x, y in zip(sa, sb):
            x.bind(y.bind_info())
            y.bind(x.bind_info())
        st = umq.jetty_pool_stats()
        assert st["total_num"] - before["total_num"] == 2 and st["sub_queues"] - before["sub_queues"] == 2 * n_sub
        # interleaved traffic on all pairs and on the main queues themselves
        for rnd in range(6):
            for i, (x, y) in enumerate(zip(sa, sb)):
                x.send(b"a%d-%d" % (i, rnd))
                y.send(b"b%d-%d" % (i, rnd) * 50)
            ma.send(b"main %d" % rnd)
            assert mb.recv() == b"main %d" % rnd
            for i, (x, y) in enumerate(zip(sa, sb)):
                assert y.recv() == b"a%d-%d" % (i, rnd)
                assert x.recv() == b"b%d-%d" % (i, rnd) * 50
        # more messages than a sub queue's window of 8: credits return per sub queue
        big = os.urandom(200_000)
        for k in range(40):
            sa[3].send(bytes([k]) * 100)
            if k % 4 == 3:
                for j in range(k - 3, k + 1):
                    assert sb[3].recv() == bytes([j]) * 100
        sa[5].send(b"small first")
        sa[5].send(big)                  # beyond the 8 KB receive buffers: pulled through a borrowed endpoint
        sa[5].send(b"small last")
        assert [sb[5].recv(), sb[5].recv(), sb[5].recv()] == [b"small first", big, b"small last"]
        assert sb[5].io_stats()["pull_rx"] == 1 and sa[5].io_stats()["pull_tx"] == 1
        assert all(q.recv(timeout_s=0.01) is None for q in sb[:4])      # nothing leaked into other sub queues
        assert sa[3].flow_control_stats()["credits_granted"] > 0
        st2 = umq.jetty_pool_stats()
        assert st2["acc_alloc_num"] - before["acc_alloc_num"] >= 6 * 2 * n_sub + 43
        assert st2["acc_alloc_num"] == st2["acc_free_num"] and st2["err_num"] == 0
        # a main queue cannot go while it has sub queues
        assert umq._lib().umq_destroy(ctypes.c_uint64(ma.h)) != 0
        assert ma.io_stats()["rx_errors"] == 0 and mb.io_stats()["rx_errors"] == 0
    finally:
        for q in made:
            q.close()
        umq.uninit()


def test_call_latency_histograms_merge_over_threads_and_restart(pair):
    """Latencies are recorded per thread: the report must add up what every thread recorded (also one that has ended
    since), and a restart must forget all of it."""
    import threading
    umq, a, b = pair
    lib = umq._lib()

    class Entry(ctypes.Structure):
        _fields_ = [(n, ctypes.c_uint64) for n in ("count", "avg_ns", "min_ns", "max_ns", "p99_ns")]
    ent = (Entry * 5)()

    def enqueue_count():
        assert lib.umq_stats_perf_get(ent) == 0
        return int(ent[0].count)   # UMQ_PERF_ENQUEUE

    got = []
    stop = threading.Event()

    def drain():                       # the receiver returns credits while the senders run
        while not stop.is_set():
            m = b.recv(timeout_s=0.05)
            if m is not None:
                got.append(m)

    rx = threading.Thread(target=drain)
    rx.start()
    try:
        assert lib.umq_stats_perf_start() == 0
        assert enqueue_count() == 0
        eagain0 = a.io_stats()["tx_eagain"]

        def sender(n):
            for i in range(n):
                a.send(b"t%d" % i)

        workers = [threading.Thread(target=sender, args=(20,)) for _ in range(3)]
        for t in workers:
            t.start()
        for t in workers:
            t.join()                   # the threads are gone: their counts must not be
        sender(5)                      # ... and this thread's come on top
        for _ in range(200):
            if len(got) >= 65:
                break
            stop.wait(0.025)
        assert len(got) == 65
        # every enqueue call is recorded, also one that found no credit and was repeated
        retried = a.io_stats()["tx_eagain"] - eagain0
        assert enqueue_count() == 65 + retried and ent[0].max_ns >= ent[0].min_ns > 0
        assert lib.umq_stats_perf_reset() == 0 and enqueue_count() == 0
        eagain1 = a.io_stats()["tx_eagain"]
        a.send(b"after")
        seen = enqueue_count()
        assert seen == 1 + a.io_stats()["tx_eagain"] - eagain1
        assert lib.umq_stats_perf_stop() == 0
        a.send(b"unseen")
        assert enqueue_count() == seen
    finally:
        stop.set()
        rx.join()
