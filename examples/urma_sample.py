#!/usr/bin/env python
"""URMA client / server sample: context -> endpoint (jetty + completion queue) -> register a segment -> exchange
segment and endpoint information over TCP -> import the peer's -> one-sided write / read, two-sided send / recv,
fetch-add -> poll completions. The same walk-through as the reference's sample program
(src/urma/examples/urma_sample.c:179-313, 773-981), through the Python binding.

    python examples/urma_sample.py --server 18515 [--dev shm0]
    python examples/urma_sample.py --client 127.0.0.1 18515 [--dev shm0]
    python examples/urma_sample.py --self          # both ends in one process
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import socket
import struct
import sys
import threading

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from umdk_b200 import urma  # noqa: E402

SEG_BYTES = 1 << 20


def exchange(sock: socket.socket, mine: bytes) -> bytes:
    sock.sendall(struct.pack("<I", len(mine)) + mine)
    n = struct.unpack("<I", _recv(sock, 4))[0]
    return _recv(sock, n)


def _recv(sock, n):
    out = b""
    while len(out) < n:
        d = sock.recv(n - len(out))
        if not d:
            raise ConnectionError("peer closed during the exchange")
        out += d
    return out


def run(sock: socket.socket, dev: str, is_client: bool) -> dict:
    ctx = urma.Context(dev)
    ep = ctx.endpoint(depth=64)
    mem = (ctypes.c_uint8 * SEG_BYTES)()
    seg = ctx.register(mem)
    peer_ep_blob = exchange(sock, ep.blob)
    peer_seg_blob = exchange(sock, seg.blob)
    peer = ctx.import_endpoint(peer_ep_blob)
    rseg = ctx.import_segment(peer_seg_blob)
    base = ctypes.addressof(mem)
    report = {}
    if is_client:
        # one-sided: write 4 KiB into the server's segment, read it back into another part of ours
        for i in range(4096):
            mem[i] = (i * 7 + 1) & 0xff
        ep.write(peer, rseg, rseg.va, base, 4096, user_ctx=1)
        ep.wait(1)
        ep.read(peer, rseg, rseg.va, base + 8192, 4096, user_ctx=2)
        ep.wait(1)
        report["write_read_ok"] = bytes(mem[0:4096]) == bytes(mem[8192:8192 + 4096])
        # atomics on a counter at offset 64 KiB of the server's segment
        olds = [ep.fetch_add(peer, rseg, rseg.va + 65536, 5) for _ in range(3)]
        report["fetch_add_olds"] = olds
        # two-sided: send a message, wait for the echo
        ep.post_recv((base + 16384, 256), user_ctx=9)
        exchange(sock, b"recv posted")
        msg = b"hello over urma"
        ctypes.memmove(base + 12288, msg, len(msg))
        ep.send(peer, base + 12288, len(msg), user_ctx=3)
        cs = ep.wait(2)     # our send completion and the echoed message
        got = [c for c in cs if c.is_recv][0]
        report["echo"] = bytes(mem[16384:16384 + got.length]).decode()
    else:
        ep.post_recv((base + 16384, 256), user_ctx=9)
        exchange(sock, b"recv posted")
        got = [c for c in ep.wait(1) if c.is_recv][0]
        ep.send(peer, base + 16384, got.length, user_ctx=4)
        ep.wait(1)
        report["served_bytes"] = got.length
        report["counter"] = struct.unpack_from("<Q", bytes(mem[65536:65536 + 8]))[0]
    exchange(sock, b"bye")
    ctx.close()
    return report


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dev", default="shm0")
    ap.add_argument("--server", type=int)
    ap.add_argument("--client", nargs=2, metavar=("HOST", "PORT"))
    ap.add_argument("--self", action="store_true", dest="both")
    a = ap.parse_args()
    if a.both:
        ls = socket.socket()
        ls.bind(("127.0.0.1", 0))
        ls.listen(1)
        res = {}
        t = threading.Thread(target=lambda: res.update(server=run(ls.accept()[0], a.dev, False)))
        t.start()
        res["client"] = run(socket.create_connection(("127.0.0.1", ls.getsockname()[1])), a.dev, True)
        t.join()
        ok = res["client"]["write_read_ok"] and res["client"]["echo"] == "hello over urma" and \
            res["client"]["fetch_add_olds"] == [0, 5, 10] and res["server"]["counter"] == 15
        print(json.dumps(dict(res, ok=ok)))
        return 0 if ok else 1
    if a.server is not None:
        ls = socket.socket()
        ls.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        ls.bind(("0.0.0.0", a.server))
        ls.listen(1)
        print(f"urma_sample server on port {a.server}", flush=True)
        print(json.dumps(run(ls.accept()[0], a.dev, False)))
        return 0
    if a.client:
        print(json.dumps(run(socket.create_connection((a.client[0], int(a.client[1]))), a.dev, True)))
        return 0
    ap.print_help()
    return 2


if __name__ == "__main__":
    sys.exit(main())
