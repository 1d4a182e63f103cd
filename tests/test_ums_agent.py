"""The UMS token agent: two daemons exchange token values over TLS on behalf of local endpoints."""
import ctypes
import os
import signal
import subprocess

import pytest

from umdk_b200 import _native

BIN = os.path.join(_native.lib_dir(), "bin", "ums_agent")
PSK = "c3" * 32


def _lib():
    lib = ctypes.CDLL(os.path.join(_native.lib_dir(), "libumdk_usock.so"))
    lib.ums_agent_put.argtypes = [ctypes.c_char_p, ctypes.c_uint64, ctypes.c_char_p, ctypes.c_uint32]
    lib.ums_agent_del.argtypes = [ctypes.c_char_p, ctypes.c_uint64]
    lib.ums_agent_get.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_char_p,
                                  ctypes.POINTER(ctypes.c_uint32)]
    lib.ums_agent_stats.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint32]
    return lib


class Agent:
    def __init__(self, tmp_path, name, args=(), env=None):
        self.sock = str(tmp_path / f"{name}.sock")
        self.proc = subprocess.Popen([BIN, "--sock", self.sock, *args], stdout=subprocess.PIPE,
                                     stderr=subprocess.STDOUT, text=True, env=dict(os.environ, **(env or {})))
        line = self.proc.stdout.readline()
        assert "listening on" in line, line + self.proc.stdout.read()
        self.banner = line
        self.addr = line.split("listening on ")[1].split(",")[0]

    def stop(self):
        self.proc.send_signal(signal.SIGTERM)
        out = self.proc.communicate(timeout=10)[0]
        return self.proc.returncode, out


def _get(lib, sock, peer, token_id):
    buf, n = ctypes.create_string_buffer(128), ctypes.c_uint32(128)
    rc = lib.ums_agent_get(sock.encode(), peer.encode() if peer else None, token_id, buf, ctypes.byref(n))
    return rc, buf.raw[:n.value] if rc == 0 else b""


def test_two_agents_exchange_tokens_over_tls(tmp_path):
    lib = _lib()
    cfg = tmp_path / "agent.conf"
    cfg.write_text(f"# agent A\npsk = {PSK}\npsk_id = ums-agents\nmax_tokens = 2   # tiny table\nlog_level = 3\n")
    a = Agent(tmp_path, "a", ["--config", str(cfg)])
    b = Agent(tmp_path, "b", env={"UMS_AGENT_PSK": PSK, "UMS_AGENT_PSK_ID": "ums-agents"})
    c = Agent(tmp_path, "c", env={"UMS_AGENT_PSK": "d4" * 32, "UMS_AGENT_PSK_ID": "ums-agents"})   # another key
    try:
        assert "pre-shared key" in a.banner
        token = os.urandom(48)
        assert lib.ums_agent_put(a.sock.encode(), 7, token, len(token)) == 0
        assert _get(lib, a.sock, None, 7) == (0, token)                    # local table
        assert _get(lib, b.sock, a.addr, 7) == (0, token)                  # B fetches it from A over TLS
        assert _get(lib, b.sock, a.addr, 7) == (0, token)                  # ... again, on the pooled connection
        assert _get(lib, b.sock, a.addr, 8)[0] == 1                        # unknown id
        assert _get(lib, b.sock, None, 7)[0] == 1                          # B itself never stored it
        assert _get(lib, c.sock, a.addr, 7)[0] == 2                        # wrong key: A refuses the handshake
        assert _get(lib, b.sock, "127.0.0.1:1", 7)[0] == 2                 # nobody listens there
        # the table is bounded; replacing a value is not a new entry; deleting frees a place
        assert lib.ums_agent_put(a.sock.encode(), 8, b"second", 6) == 0
        assert lib.ums_agent_put(a.sock.encode(), 9, b"third", 5) == 4
        assert lib.ums_agent_put(a.sock.encode(), 8, b"second'", 7) == 0
        assert lib.ums_agent_del(a.sock.encode(), 7) == 0 and lib.ums_agent_del(a.sock.encode(), 7) == 1
        assert lib.ums_agent_put(a.sock.encode(), 9, b"third", 5) == 0
        assert _get(lib, b.sock, a.addr, 7)[0] == 1 and _get(lib, b.sock, a.addr, 8) == (0, b"second'")
        text = ctypes.create_string_buffer(160)
        assert lib.ums_agent_stats(a.sock.encode(), text, 160) == 0
        sa = dict(zip(text.value.decode().split()[0::2], text.value.decode().split()[1::2]))
        assert sa["tok"] == "2" and sa["srv"] == "5" and sa["tls"] == "1/1"
        assert lib.ums_agent_stats(b.sock.encode(), text, 160) == 0
        sb = dict(zip(text.value.decode().split()[0::2], text.value.decode().split()[1::2]))
        assert sb["fwd"] == "6" and sb["perr"] == "1" and sb["pool"].startswith("1/1/")   # one dial, then reuse
        assert lib.ums_agent_get(b"/nonexistent/agent.sock", None, 1, text, ctypes.byref(ctypes.c_uint32(128))) == -1
        admin = subprocess.run([os.path.join(_native.lib_dir(), "bin", "ums_admin"), "agent", a.sock],
                               capture_output=True, text=True, timeout=10)
        assert admin.returncode == 0 and "tokens stored" in admin.stdout and "lookups served to peers" in admin.stdout
        rows = dict(line.rsplit(None, 1) for line in admin.stdout.strip().splitlines())
        assert rows["lookups served to peers"] == "5" and rows["TLS accepted/refused"] == "1/1"
    finally:
        results = [x.stop() for x in (a, b, c)]
    for rc, out in results:
        assert rc == 0 and "ums_agent: stopped" in out, out
    assert not os.path.exists(a.sock)                                      # removed on the way out


def test_agent_refuses_bad_configuration(tmp_path):
    def run(args, env=None):
        e = {k: v for k, v in os.environ.items() if not k.startswith("UMS_AGENT_")}
        e.update(env or {})
        p = subprocess.run([BIN, "--sock", str(tmp_path / "x.sock"), *args], capture_output=True, text=True, env=e,
                           timeout=10)
        return p.returncode, p.stdout + p.stderr
    rc, out = run([])
    assert rc != 0 and "no key or certificates" in out
    rc, out = run([], {"UMS_AGENT_PSK": "zz"})
    assert rc != 0 and "malformed" in out
    cfg = tmp_path / "bad.conf"
    cfg.write_text("psk = " + PSK + "\nports = 99\n")
    rc, out = run(["--config", str(cfg)])
    assert rc != 0 and "line 2" in out and "unknown key" in out
    cfg.write_text("psk = " + PSK + "\nport = seventy\n")
    rc, out = run(["--config", str(cfg)])
    assert rc != 0 and "bad value for port" in out
    cfg.write_text("tls_ca = /tmp/ca.pem\n")
    rc, out = run(["--config", str(cfg)])
    assert rc != 0 and "go together" in out


def test_ums_connection_setup_through_the_agents(tmp_path):
    """With UMS_AGENT_SOCK / UMS_AGENT_ADDR the connecting side leaves the ring name with its agent and the accepting
    side has its own agent fetch it: the connection is accelerated, the agents' counters show the exchange, and a
    server without an agent declines (plain TCP, stream intact)."""
    import sys
    lib_path = os.path.join(_native.lib_dir(), "libumdk_usock.so")
    server = tmp_path / "srv.py"
    server.write_text(
        "import socket\n"
        "ls = socket.socket(); ls.bind(('127.0.0.1', 0)); ls.listen(4)\n"
        "print(ls.getsockname()[1], flush=True)\n"
        "c, _ = ls.accept()\n"
        "while True:\n"
        "    d = c.recv(65536)\n"
        "    if not d: break\n"
        "    c.sendall(d)\n"
        "c.close()\n")
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
        f"lib = ctypes.CDLL({lib_path!r})\n"
        "st = (ctypes.c_uint64 * 18)(); lib.ums_get_stats(st)\n"
        "print('STATS ums=%d fallback=%d auth_fail=%d' % (st[0], st[1], st[8]))\n")
    wrapper = os.path.join(os.path.dirname(_native.lib_dir()), "bin", "ums_run")
    base = {k: v for k, v in os.environ.items() if not k.startswith("UMS_")}
    base.update(URMA_SHM_DIR=str(tmp_path / "urma"), UMS_SHM_DIR=str(tmp_path / "ums"))
    env_agents = {"UMS_AGENT_PSK": PSK}
    a, b = Agent(tmp_path, "cli_agent", env=env_agents), Agent(tmp_path, "srv_agent", env=env_agents)
    lib = _lib()

    def stats(agent):
        text = ctypes.create_string_buffer(160)
        assert lib.ums_agent_stats(agent.sock.encode(), text, 160) == 0
        words = text.value.decode().split()
        return dict(zip(words[0::2], words[1::2]))

    def run_pair(server_env):
        srv = subprocess.Popen([wrapper, sys.executable, str(server)], stdout=subprocess.PIPE, text=True,
                               env=dict(base, **server_env))
        try:
            port = srv.stdout.readline().strip()
            r = subprocess.run([wrapper, sys.executable, str(client), port], capture_output=True, text=True, timeout=60,
                               env=dict(base, UMS_AGENT_SOCK=a.sock, UMS_AGENT_ADDR=a.addr))
            assert r.returncode == 0, r.stdout + r.stderr
            srv.wait(timeout=30)
            return r.stdout.strip().splitlines()[-1]
        finally:
            if srv.poll() is None:
                srv.kill()
    try:
        assert run_pair({"UMS_AGENT_SOCK": b.sock}) == "STATS ums=1 fallback=0 auth_fail=0"
        sa, sb = stats(a), stats(b)
        assert sa["put"] == "1" and sa["del"] == "1" and sa["srv"] == "1" and sa["tok"] == "0"   # stored, served, removed
        assert sb["fwd"] == "1" and sb["perr"] == "0"
        # a server that has no agent cannot resolve the reference: it declines and the client stays on TCP
        assert run_pair({}) == "STATS ums=0 fallback=1 auth_fail=0"
        assert stats(a)["put"] == "2" and stats(a)["srv"] == "1"
    finally:
        for x in (a, b):
            x.stop()


def test_sample_configuration_parses(tmp_path):
    """The sample configuration shipped beside the unit file uses only keys the daemon knows (it stops at the missing
    certificate files, not at the parser)."""
    sample = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "ums_agent",
                          "ums_agent.conf")
    text = open(sample).read().replace("/run/umdk/ums_agent.sock", str(tmp_path / "s.sock")).replace("7471", "0")
    cfg = tmp_path / "sample.conf"
    cfg.write_text(text)
    env = {k: v for k, v in os.environ.items() if not k.startswith("UMS_AGENT_")}
    p = subprocess.Popen([BIN, "--config", str(cfg), "--ip", "127.0.0.1"], stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True, env=env)
    line = p.stdout.readline()
    try:
        assert "listening on 127.0.0.1:" in line and "certificates" in line, line
    finally:
        p.send_signal(signal.SIGTERM)
        p.communicate(timeout=10)
    assert p.returncode == 0
