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
