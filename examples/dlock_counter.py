#!/usr/bin/env python
"""DLock sample: several client threads increment a shared counter under a distributed lock and, separately, with the
server-side 64-bit atomic object; both must end at threads x increments. Counterpart of the reference's dlock example
(src/ulock/dlock/examples).

    python examples/dlock_counter.py [--threads N] [--increments N] [--fair] [--psk HEX]
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from umdk_b200 import dlock  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--threads", type=int, default=4)
    ap.add_argument("--increments", type=int, default=200)
    ap.add_argument("--fair", action="store_true")
    ap.add_argument("--psk", default="")
    a = ap.parse_args()
    if a.psk:
        dlock.set_psk(a.psk, "dlock-counter")
    srv = dlock.Server()
    plain = [0]            # protected only by the distributed lock

    def worker():
        c = dlock.Client(srv.ip, srv.port)
        lk = c.get_lock("counter", dlock.FAIR if a.fair else dlock.ATOMIC)
        obj = c.atomic_get("hits")
        for _ in range(a.increments):
            c.lock(lk, expire_ms=5000, timeout_ms=20000)
            plain[0] += 1
            c.unlock(lk)
            c.atomic_faa(obj, 1)
        c.close()

    boot = dlock.Client(srv.ip, srv.port)
    obj = boot.atomic_create("hits", 0)
    ts = [threading.Thread(target=worker) for _ in range(a.threads)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    hits = boot.atomic_snapshot(obj)
    st = srv.stats()
    boot.close()
    srv.stop()
    want = a.threads * a.increments
    ok = plain[0] == want and hits == want
    print(json.dumps({"ok": ok, "locked_counter": plain[0], "atomic_counter": hits, "want": want,
                      "trylock_ok": st["trylock_ok"], "trylock_busy": st["trylock_busy"]}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
