#!/usr/bin/env python
"""URPC sample: a server registers two functions, a client attaches a channel and calls them synchronously and
asynchronously; optional pre-shared key (TLS 1.3 handshake + sealed payloads). Counterpart of the reference's
framework example (src/urpc/examples/framework).

    python examples/urpc_echo.py [--psk HEX] [--calls N]
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from umdk_b200 import urpc  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--psk", default="")
    ap.add_argument("--calls", type=int, default=200)
    a = ap.parse_args()
    if a.psk:
        urpc.set_psk(a.psk, "urpc-echo")
    urpc.init(default_timeout_ms=3000)
    srv = urpc.Server()
    srv.register(1, lambda b: b)                       # echo
    srv.register(2, lambda b: str(len(b)).encode())    # length
    ch = urpc.Channel(srv.ip, srv.port)
    ok = ch.call(1, b"ping") == b"ping" and ch.call(2, b"x" * 1000) == b"1000"
    t0 = time.perf_counter()
    for i in range(a.calls):
        ok &= ch.call(1, i.to_bytes(4, "little")) == i.to_bytes(4, "little")
    dt = time.perf_counter() - t0
    for i in range(16):
        ch.call_async(1, bytes([i]), user_ctx=i)
    done = {}
    deadline = time.monotonic() + 5
    while len(done) < 16 and time.monotonic() < deadline:
        for _ev, ctx, status, data in ch.poll():
            done[ctx] = (status, data)
    ok &= done == {i: (0, bytes([i])) for i in range(16)}
    st = urpc.stats()
    sessions = urpc.admin_query("sessions").strip()
    ch.close()
    srv.stop()
    urpc.uninit()
    print(json.dumps({"ok": bool(ok), "sync_calls_per_s": round(a.calls / dt), "calls": st["calls"],
                      "responses": st["responses"], "sessions": sessions}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
