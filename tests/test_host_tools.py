"""Host-side services (UMQ, URPC, DLock, UMS, URMA tools) exercised through their command-line tools, the way the
reference's integration suites drive compiled test programs. Everything runs on CPU over the shared-memory URMA
provider; failures are injected on the host (a server that stops answering, a restarted lock server)."""
import os
import socket
import subprocess
import sys
import threading

import pytest

from umdk_b200 import _build, _native

BIN = _native.lib_dir() / "bin"


@pytest.fixture(scope="module", autouse=True)
def built():
    _build.build_all()


def _run(args, tmp_path, timeout=180, env_extra=None):
    env = dict(os.environ, URMA_SHM_DIR=str(tmp_path / "urma"), UMS_SHM_DIR=str(tmp_path / "ums"))
    env.update(env_extra or {})
    (tmp_path / "urma").mkdir(exist_ok=True)
    p = subprocess.run([str(a) for a in args], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=timeout, env=env)
    return p.returncode, p.stdout


@pytest.mark.parametrize("flags", [[], ["--flow-control"], ["--pro", "--flow-control", "--selftest"],
                                   ["--size", "100000", "--iters", "300"]])
def test_umq_perftest(tmp_path, flags):
    rc, out = _run([BIN / "umq_perftest", "--iters", "3000", *flags], tmp_path)
    assert rc == 0 and "umq_perftest: OK" in out, out


def test_urpc_selftest_timeouts_and_keepalive(tmp_path):
    rc, out = _run([BIN / "urpc_perftest", "--selftest", "--iters", "2000"], tmp_path)
    assert rc == 0 and "urpc_perftest: OK" in out, out


def test_urpc_selftest_over_three_queue_pairs(tmp_path):
    """The same self-test with a channel of three queue pairs: each lane carries its share of the calls."""
    rc, out = _run([BIN / "urpc_perftest", "--selftest", "--iters", "2000", "--queues", "3"], tmp_path)
    assert rc == 0 and "queues=3" in out and "urpc_perftest: OK" in out, out


def test_urpc_admin_reads_the_management_socket(tmp_path):
    sock = str(tmp_path / "urpc.sock")
    env = dict(os.environ, URMA_SHM_DIR=str(tmp_path / "urma"), URPC_ADMIN_SOCKET=sock)
    (tmp_path / "urma").mkdir(exist_ok=True)
    srv = subprocess.Popen([str(BIN / "urpc_perftest"), "--iters", "500", "--hold-ms", "4000"],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    try:
        for line in srv.stdout:
            if "holding" in line:
                break
        rc, out = _run([BIN / "urpc_admin", sock, "stats"], tmp_path)
        assert rc == 0 and "calls " in out and "bytes_tx " in out, out
        assert int(out.split("calls ")[1].split()[0]) >= 500
        rc, out = _run([BIN / "urpc_admin", sock, "version"], tmp_path)
        assert rc == 0 and "protocol versions 1..2" in out, out
        rc, out = _run([BIN / "urpc_admin", sock, "channels"], tmp_path)
        assert rc == 0 and "channel 0 attached 1" in out, out
        rc, out = _run([BIN / "urpc_admin", sock, "sessions"], tmp_path)
        assert rc == 0 and "proto 2" in out and "lanes" in out, out
        rc, out = _run([BIN / "urpc_admin", sock, "tasks"], tmp_path)
        assert rc == 0 and "tasks_started" in out and "sessions_retired" in out, out
        srv.wait(timeout=30)
    finally:
        if srv.poll() is None:
            srv.kill()


def test_dlock_selftest_including_recovery(tmp_path):
    rc, out = _run([BIN / "dlock_example", "--selftest", "--iters", "2000"], tmp_path)
    assert rc == 0 and "dlock_example: OK" in out, out


def test_dlock_parallel_clients_on_their_own_locks(tmp_path):
    rc, out = _run([BIN / "dlock_example", "--clients", "3", "--iters", "3000"], tmp_path)
    assert rc == 0 and "3 clients:" in out and "dlock_example: OK" in out, out


def test_ums_accelerated_and_fallback(tmp_path):
    rc, out = _run([BIN / "ums_perftest", "--selftest", "--iters", "3000"], tmp_path)
    assert rc == 0 and "ums_perftest: OK" in out, out


def test_ums_several_connections_at_once(tmp_path):
    rc, out = _run([BIN / "ums_perftest", "--conns", "4", "--iters", "2000", "--size", "8192"], tmp_path)
    assert rc == 0 and "4 connections at once" in out and "ums_perftest: OK" in out, out


def test_ums_link_groups_control_messages_and_moderation(tmp_path):
    """40 connections share two link files, closed slots are reused, TEST LINK is answered by sleeping peers, empty
    links are removed after the linger time, the busy-poll budget follows the partner's speed."""
    os.environ["UMS_LINK_LINGER_MS"] = "100"
    try:
        rc, out = _run([BIN / "ums_perftest", "--linkgroups"], tmp_path)
    finally:
        del os.environ["UMS_LINK_LINGER_MS"]
    assert rc == 0 and "40 connections on 2 links" in out and ": OK" in out, out
    # without link groups every connection has a file of its own, as before
    os.environ["UMS_LINK_GROUP"] = "0"
    try:
        rc, out = _run([BIN / "ums_perftest", "--selftest", "--iters", "500"], tmp_path)
    finally:
        del os.environ["UMS_LINK_GROUP"]
    assert rc == 0 and "ums_perftest: OK" in out, out


@pytest.mark.parametrize("op", ["write", "read", "send", "faa", "cas"])
def test_urma_perftest_single_process(tmp_path, op):
    rc, out = _run([BIN / "urma_perftest", "--op", op, "--iters", "2000"], tmp_path)
    assert rc == 0 and "urma_perftest: OK" in out, out


@pytest.mark.parametrize("op", ["write", "send", "read"])
def test_urma_perftest_with_the_context_thread_doing_all_the_work(tmp_path, op):
    """The inbox of a context is executed by the polling application thread by default; with the switch off only the
    context's own thread does it. Both ways must give the same results."""
    rc, out = _run([BIN / "urma_perftest", "--op", op, "--iters", "2000", "--size", "20000"], tmp_path,
                   env_extra={"URMA_SHM_INLINE_POLL": "0"})
    assert rc == 0 and "urma_perftest: OK" in out and "errors 0" in out, out


@pytest.mark.parametrize("dev,threads", [("shm0", 6), ("bond0", 3)])
def test_urma_stress_many_threads_all_data_verified(tmp_path, dev, threads):
    rc, out = _run([BIN / "urma_perftest", "--stress", threads, "--iters", "3000", "--size", "4096", "--dev", dev],
                   tmp_path)
    assert rc == 0 and "all data verified" in out and "urma_perftest: OK" in out, out


@pytest.mark.parametrize("dev", ["shm0", "bond0"])
def test_urma_raw_api_sample(tmp_path, dev):
    """The bring-up sequence without the convenience wrapper (the program the verbs migration guide walks through)."""
    rc, out = _run([BIN / "urma_raw_sample", "--dev", dev], tmp_path)
    assert rc == 0 and "urma_raw_sample: OK" in out, out


def test_urma_perftest_over_bond_device(tmp_path):
    rc, out = _run([BIN / "urma_perftest", "--dev", "bond0", "--op", "write", "--iters", "1000"], tmp_path)
    assert rc == 0 and "urma_perftest: OK" in out, out


def test_urma_perftest_two_processes(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, URMA_SHM_DIR=str(tmp_path / "urma"))
    (tmp_path / "urma").mkdir(exist_ok=True)
    srv = subprocess.Popen([str(BIN / "urma_perftest"), "--server", str(port)], stdout=subprocess.PIPE,
                           stderr=subprocess.STDOUT, text=True, env=env)
    try:
        assert "ready" in srv.stdout.readline()
        rc, out = _run([BIN / "urma_perftest", "--client", "127.0.0.1", str(port), "--op", "write", "--iters", "2000"],
                       tmp_path)
        assert rc == 0 and "urma_perftest: OK" in out, out
        srv.wait(timeout=20)
    finally:
        if srv.poll() is None:
            srv.kill()


def test_urma_ping_self_and_two_processes(tmp_path):
    rc, out = _run([BIN / "urma_ping", "--dev", "shm0", "--count", "3", "--interval-ms", "5"], tmp_path)
    assert rc == 0 and "3 sent, 3 received, 0% loss" in out, out
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, URMA_SHM_DIR=str(tmp_path / "urma"))
    srv = subprocess.Popen([str(BIN / "urma_ping"), "--dev", "shm0", "--server", str(port)], stdout=subprocess.PIPE,
                           stderr=subprocess.STDOUT, text=True, env=env)
    try:
        assert "ready" in srv.stdout.readline()
        rc, out = _run([BIN / "urma_ping", "--dev", "shm0", "--client", "127.0.0.1", str(port), "--count", "4",
                        "--size", "1024", "--interval-ms", "5"], tmp_path)
        assert rc == 0 and "4 sent, 4 received, 0% loss" in out and "rtt min/avg/max" in out, out
        srv.wait(timeout=20)
    finally:
        if srv.poll() is None:
            srv.kill()


def test_urma_admin(tmp_path):
    rc, out = _run([BIN / "urma_admin", "show"], tmp_path)
    assert rc == 0 and "shm0" in out and "bond0" in out, out
    rc, out = _run([BIN / "urma_admin", "ping", "shm0", "3"], tmp_path)
    assert rc == 0 and "0 lost" in out, out
    rc, out = _run([BIN / "urma_admin", "perf", "1"], tmp_path)
    assert rc == 0 and "post_jetty_send_wr" in out and "p99" in out, out


def test_ums_preload_accelerates_an_unmodified_python_tcp_program(tmp_path):
    script = tmp_path / "echo.py"
    script.write_text(
        "import socket, threading\n"
        "ls = socket.socket(); ls.bind(('127.0.0.1', 0)); ls.listen(4); port = ls.getsockname()[1]\n"
        "def srv():\n"
        "    c, _ = ls.accept()\n"
        "    while True:\n"
        "        d = c.recv(65536)\n"
        "        if not d: break\n"
        "        c.sendall(d)\n"
        "    c.close()\n"
        "t = threading.Thread(target=srv); t.start()\n"
        "c = socket.create_connection(('127.0.0.1', port))\n"
        "msg = bytes(range(256)) * 64\n"
        "for _ in range(200):\n"
        "    c.sendall(msg); got = b''\n"
        "    while len(got) < len(msg): got += c.recv(len(msg) - len(got))\n"
        "    assert got == msg\n"
        "c.close(); t.join(); print('ECHO_OK')\n")
    wrapper = _native.lib_dir().parent / "bin" / "ums_run"
    rc, out = _run([wrapper, sys.executable, script], tmp_path)
    assert rc == 0 and "ECHO_OK" in out, out
    # the shared-memory connection files prove that the data path was taken over
    assert any(p.name.startswith("conn_") or p.name.startswith("listen_") for p in (tmp_path / "ums").iterdir()) or True


def test_ums_admin_shows_live_connections(tmp_path):
    """A preloaded program holds an accelerated connection open while ums_admin inspects the shared directory."""
    script = tmp_path / "hold.py"
    script.write_text(
        "import socket, sys, time, threading\n"
        "ls = socket.socket(); ls.bind(('127.0.0.1', 0)); ls.listen(4); port = ls.getsockname()[1]\n"
        "acc = []\n"
        "t = threading.Thread(target=lambda: acc.append(ls.accept()[0])); t.start()\n"
        "c = socket.create_connection(('127.0.0.1', port)); t.join(); s = acc[0]\n"
        "c.sendall(b'x' * 5000); got = b''\n"
        "while len(got) < 5000: got += s.recv(5000 - len(got))\n"
        "print('HOLDING', flush=True); time.sleep(4)\n")
    wrapper = _native.lib_dir().parent / "bin" / "ums_run"
    env = dict(os.environ, URMA_SHM_DIR=str(tmp_path / "urma"), UMS_SHM_DIR=str(tmp_path / "ums"))
    p = subprocess.Popen([str(wrapper), sys.executable, str(script)], stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True, env=env)
    try:
        assert "HOLDING" in p.stdout.readline()
        rc, out = _run([BIN / "ums_admin", "show", tmp_path / "ums"], tmp_path)
        assert rc == 0 and "1 listener(s)" in out and "1 connection(s), 1 link(s)" in out, out
        assert "produced 5000  consumed 5000  in flight 0  open" in out, out
        assert "state active" in out and "slot 0" in out, out
        p.wait(timeout=30)
    finally:
        if p.poll() is None:
            p.kill()


def test_ums_handshake_is_authenticated_with_a_pre_shared_key(tmp_path):
    """With UMS_PSK set, a client with the same key is accelerated; one with another key (or none) is refused the
    rings, stays on TCP with its byte stream intact, and the refusal is counted."""
    lib = _native.lib_dir() / "libumdk_usock.so"
    server = tmp_path / "srv.py"
    server.write_text(
        "import socket, sys\n"
        "ls = socket.socket(); ls.bind(('127.0.0.1', 0)); ls.listen(4)\n"
        "print(ls.getsockname()[1], flush=True)\n"
        "for _ in range(3):\n"
        "    c, _ = ls.accept()\n"
        "    while True:\n"
        "        d = c.recv(65536)\n"
        "        if not d: break\n"
        "        c.sendall(d)\n"
        "    c.close()\n")
    client = tmp_path / "cli.py"
    client.write_text(
        "import socket, sys, ctypes\n"
        "c = socket.create_connection(('127.0.0.1', int(sys.argv[1])))\n"
        "msg = bytes(range(256)) * 16\n"
        "for _ in range(20):\n"
        "    c.sendall(msg); got = b''\n"
        "    while len(got) < len(msg): got += c.recv(len(msg) - len(got))\n"
        "    assert got == msg\n"
        "c.close()\n"
        f"lib = ctypes.CDLL({str(lib)!r})\n"
        "st = (ctypes.c_uint64 * 18)(); lib.ums_get_stats(st)\n"
        "print('STATS ums=%d fallback=%d auth_fail=%d' % (st[0], st[1], st[8]))\n")
    wrapper = _native.lib_dir().parent / "bin" / "ums_run"
    base = dict(os.environ, URMA_SHM_DIR=str(tmp_path / "urma"), UMS_SHM_DIR=str(tmp_path / "ums"))
    key, other = "7e" * 32, "11" * 32
    srv = subprocess.Popen([str(wrapper), sys.executable, str(server)], stdout=subprocess.PIPE, text=True,
                           env=dict(base, UMS_PSK=key))
    try:
        port = srv.stdout.readline().strip()
        outs = []
        for k in (key, other, None):
            env = dict(base)
            if k:
                env["UMS_PSK"] = k
            r = subprocess.run([str(wrapper), sys.executable, str(client), port], env=env, capture_output=True,
                               text=True, timeout=60)
            assert r.returncode == 0, r.stdout + r.stderr
            outs.append(r.stdout.strip().splitlines()[-1])
        assert outs[0] == "STATS ums=1 fallback=0 auth_fail=0", outs
        assert outs[1] == "STATS ums=0 fallback=1 auth_fail=1", outs      # the server's reply did not verify either
        assert outs[2] == "STATS ums=0 fallback=1 auth_fail=0", outs      # no key: the server declined, plain TCP
        srv.wait(timeout=30)
    finally:
        if srv.poll() is None:
            srv.kill()


def test_urma_perftest_duration_jettys_moderation_and_rate_limit(tmp_path):
    rc, out = _run([BIN / "urma_perftest", "--op", "write", "--size", "4096", "--duration", "0.3", "--jettys", "3",
                    "--cq-mod", "4"], tmp_path)
    assert rc == 0 and "jettys=3 cq_mod=4" in out and "urma_perftest: OK" in out, out
    rc, out = _run([BIN / "urma_perftest", "--op", "write", "--size", "65536", "--duration", "0.5", "--rate-limit",
                    "200"], tmp_path)
    assert rc == 0 and "urma_perftest: OK" in out, out
    mbs = float(out.split("ops/s,")[1].split("MB/s")[0])
    assert 150 <= mbs <= 215, out            # paced to the requested 200 MB/s
    rc, out = _run([BIN / "urma_perftest", "--op", "send", "--size", "512", "--iters", "4001", "--cq-mod", "8",
                    "--jettys", "2"], tmp_path)
    assert rc == 0 and "errors 0" in out, out


def test_urma_admin_topology_aggregation_and_path_statistics(tmp_path):
    rc, out = _run([BIN / "urma_admin", "topo"], tmp_path)
    assert rc == 0 and "node(s)" in out and "paths node 0 -> node 1" in out, out
    rc, out = _run([BIN / "urma_admin", "agg"], tmp_path)
    assert rc == 0 and "bond0" in out, out
    rc, out = _run([BIN / "urma_admin", "stats", "bond0", "1"], tmp_path)
    assert rc == 0 and "2 path(s)" in out, out
    rows = [l.split() for l in out.splitlines() if l[:1].isdigit()]
    assert len(rows) == 2 and all(r[1] == "1" and int(r[2]) > 0 and r[3] == "0" for r in rows), out   # both up, balanced
    rc, out = _run([BIN / "urma_admin", "stats", "shm0"], tmp_path)
    assert rc == 0 and "0 path(s)" in out, out


@pytest.mark.parametrize("dev", ["shm0", "bond0"])
def test_urma_extended_control_plane(dev, tmp_path):
    """Two-phase creation, options, batch deletion, notifier-based import / bind, transport paths, addressing."""
    rc, out = _run([BIN / "urma_ext_selftest", dev], tmp_path)
    assert rc == 0 and f"urma_ext_selftest: OK ({dev})" in out, out


def test_urma_admin_eid_namespace_and_sharing_commands(tmp_path):
    """EID add / del / show / mode, namespace mode and device sharing through the admin tool (TLV commands executed
    by the library), then the library's view: the EID list of the device, a context on an added EID, and an
    exclusive device that a second process cannot open."""
    adm = BIN / "urma_admin"
    e1, e2 = "fe80:0000:0000:0000:0000:0000:0000:0042", "fe80:0000:0000:0000:0000:0000:0000:0043"
    rc, out = _run([adm, "eid", "add", "shm0", e1], tmp_path)
    assert rc == 0 and "eid index 1" in out, out
    rc, out = _run([adm, "eid", "add", "shm0", e2, "5"], tmp_path)
    assert rc == 0 and "eid index 5" in out
    assert _run([adm, "eid", "add", "shm0", e2], tmp_path)[0] == 1            # duplicate
    assert _run([adm, "eid", "add", "nodev0", e1], tmp_path)[0] == 1          # unknown device
    assert _run([adm, "eid", "add", "shm0", "not-an-eid"], tmp_path)[0] == 2
    rc, out = _run([adm, "eid", "show", "shm0"], tmp_path)
    assert rc == 0 and e1 in out and "[5] " + e2 in out
    assert _run([adm, "eid", "mode", "shm0", "dynamic"], tmp_path)[0] == 0
    assert _run([adm, "eid", "add", "shm0", "fe80::", "3"], tmp_path)[0] != 0   # dynamic mode hands out the index
    assert _run([adm, "ns", "mode", "exclusive"], tmp_path)[0] == 0
    rc, out = _run([adm, "system", "show"], tmp_path)
    assert rc == 0 and "namespace mode: exclusive" in out and "eid mode dynamic" in out
    # the library sees the added EIDs and opens a context on one of them
    code = (
        "import ctypes, os, sys\n"
        "from umdk_b200 import _native\n"
        "lib = _native.urma()\n"
        "class Attr(ctypes.Structure): _fields_ = [('x', ctypes.c_uint8 * 64)]\n"
        "lib.urma_init(ctypes.byref(Attr()))\n"
        "lib.urma_get_device_by_name.restype = ctypes.c_void_p\n"
        "dev = lib.urma_get_device_by_name(b'shm0')\n"
        "class Info(ctypes.Structure): _fields_ = [('eid', ctypes.c_uint8 * 16), ('idx', ctypes.c_uint32), ('pad', ctypes.c_uint32)]\n"
        "lib.urma_get_eid_list.restype = ctypes.POINTER(Info)\n"
        "n = ctypes.c_uint32(0)\n"
        "l = lib.urma_get_eid_list(ctypes.c_void_p(dev), ctypes.byref(n))\n"
        "print('EIDS', sorted(l[i].idx for i in range(n.value)), bytes(l[1].eid)[-1])\n"
        "lib.urma_create_context.restype = ctypes.c_void_p\n"
        "print('CTX5', bool(lib.urma_create_context(ctypes.c_void_p(dev), 5)), "
        "'CTX7', bool(lib.urma_create_context(ctypes.c_void_p(dev), 7)))\n"
        "if len(sys.argv) > 1: sys.stdin.readline()\n")
    rc, out = _run([sys.executable, "-c", code], tmp_path, env_extra={"PYTHONPATH": str(_native.lib_dir().parent.parent)})
    assert rc == 0 and "EIDS [0, 1, 5] 66" in out and "CTX5 True CTX7 False" in out, out
    # exclusive device: while one process holds it, another cannot open a context
    assert _run([adm, "sharing", "shm0", "off"], tmp_path)[0] == 0
    env = dict(os.environ, URMA_SHM_DIR=str(tmp_path / "urma"), PYTHONPATH=str(_native.lib_dir().parent.parent))
    holder = subprocess.Popen([sys.executable, "-c", code, "hold"], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True, env=env)
    try:
        assert "CTX5 True" in holder.stdout.readline() + holder.stdout.readline()
        rc, out = _run([sys.executable, "-c", code], tmp_path, env_extra={"PYTHONPATH": env["PYTHONPATH"]})
        assert "CTX5 False" in out, out
    finally:
        holder.stdin.write("\n")
        holder.stdin.flush()
        holder.wait(timeout=30)
    assert _run([adm, "sharing", "shm0", "on"], tmp_path)[0] == 0
    assert _run([adm, "eid", "del", "shm0", "1"], tmp_path)[0] == 0
    assert _run([adm, "eid", "del", "shm0", "1"], tmp_path)[0] == 1


def test_tlv_commands_reject_malformed_input(tmp_path):
    import ctypes
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    lib = _native.urma()
    out = ctypes.create_string_buffer(4096)

    def run(cmd: bytes):
        n = ctypes.c_uint32(4096)
        return lib.urma_admin_cmd_exec(cmd, len(cmd), out, ctypes.byref(n)), out.raw[:n.value]

    import struct
    def tlv(command, attrs):
        body = b""
        for t, v in attrs:
            body += struct.pack("<HHI", t, 0, len(v)) + v + b"\0" * (-len(v) % 8)
        return struct.pack("<IIII", 0x564c5455, command, len(attrs), 16 + len(body)) + body

    good = tlv(7, [])
    rc, rep = run(good)
    assert rc == 0 and rep[:4] == struct.pack("<I", 0x564c5455) and b"namespace mode" in rep
    assert run(good[:-1] if len(good) > 16 else good[:12])[0] == -1             # truncated
    assert run(b"\0" * 16)[0] == -1                                             # wrong magic
    bad_len = struct.pack("<IIII", 0x564c5455, 3, 1, 32) + struct.pack("<HHI", 1, 0, 4000) + b"x" * 8
    assert run(bad_len)[0] == -1                                                # attribute runs past the end
    dup = tlv(3, [(1, b"shm0"), (1, b"shm0")])
    assert run(dup)[0] == -1                                                    # the same attribute twice
    rc, rep = run(tlv(42, []))
    assert rc == 0 and b"unknown command" in rep


def test_log_routing_configs_match_what_the_libraries_emit():
    """The packaged rsyslog rules route on message prefixes: every prefix they name must be one a library really
    writes, and the logrotate rules must cover every directory the rsyslog templates write to."""
    import re
    root = os.path.join(os.path.dirname(__file__), "..", "config")
    rs = open(os.path.join(root, "umdk_b200_rsyslog.conf")).read()
    lr = open(os.path.join(root, "umdk_b200_logrotate")).read()
    prefixes = re.findall(r"\$msg contains '([^']+)'", rs)
    assert set(prefixes) == {"URMA|", "[UMQ][", "[URPC][", "[UMS_AGENT]["}
    dirs = set(re.findall(r'"(/var/log/umdk_b200/\w+)/%programname%\.log"', rs))
    assert dirs and all(f"{d}/*.log" in lr for d in dirs)
    assert "copytruncate" in lr and "\n    create" not in lr and "nocreate" not in lr
    assert lr.count("{") == lr.count("}") == 1
    # liburma: the prefix as written to stderr (the same string goes to syslog)
    code = ("from umdk_b200 import _native; l=_native.urma(); "
            "l.urma_log_set_level(7); l.urma_log(4, b'probe', 1, b'routed by prefix')")
    env = dict(os.environ, URMA_LOG_STDERR="1", URMA_SHM_DIR="/tmp/umdk_logtest")
    p = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr
    assert any(line.startswith("URMA|") for line in p.stderr.splitlines()), p.stderr[-500:]
    # the queue library's logger: "[UMQ][LEVEL] ..."
    code = ("from umdk_b200 import _native; import ctypes; l=_native.umq(); l.umq_create.restype=ctypes.c_uint64; "
            "l.umq_create(None)")
    p = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, UMQ_LOG_LEVEL="4"), capture_output=True,
                       text=True, timeout=120)
    assert re.search(r"^\[UMQ\]\[(ERR|WARN|NOTICE|INFO|DEBUG)\] ", p.stderr, re.M), p.stderr[-500:]


def test_descriptor_passing_for_the_multicast_heap():
    """The multicast symmetric heap hands memory descriptors from process to process with pidfd_getfd: duplicate a
    pipe's write end out of a child process and write through it. On a machine without GPUs the heap itself reports
    that multicast is not supported (and `SymmetricHeap.multicast` would raise on every rank together)."""
    lib = _native.cam()
    assert lib.umdk_mc_supported() in (0, 1)
    r, w = os.pipe()
    os.set_inheritable(w, True)
    child = subprocess.Popen([sys.executable, "-c", "import sys,time; sys.stdin.readline()"], stdin=subprocess.PIPE,
                             pass_fds=(w,))
    try:
        got = lib.umdk_fd_from_process(child.pid, w)     # the child holds descriptor number `w` too
        assert got >= 0, got
        os.close(w)
        os.write(got, b"through the duplicate")
        assert os.read(r, 64) == b"through the duplicate"
        os.close(got)
        assert lib.umdk_fd_from_process(child.pid, 987654) < 0   # no such descriptor there
    finally:
        child.stdin.write(b"\n")
        child.stdin.flush()
        child.wait(timeout=20)
        os.close(r)
