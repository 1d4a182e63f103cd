#!/usr/bin/env python
"""URPC sample: queue pairs that join and leave an ATTACHED channel, acknowledgements for deferred requests, and
the server's notice when its function table changes (all of it protocol version 2; the attach negotiates the
version, so the same script reports "version 1" and skips these parts against an old server).

    python examples/urpc_live_queues.py [--calls N]
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
    ap.add_argument("--calls", type=int, default=60)
    a = ap.parse_args()
    urpc.init(default_timeout_ms=3000)
    srv = urpc.Server()
    srv.register(1, lambda b: b[::-1])
    srv.deferred = lambda fid, args: b"deferred:" + args      # functions without a registered handler land here
    ch = urpc.Channel(srv.ip, srv.port)
    version, caps = ch.protocol()
    ok = ch.call(1, b"abc") == b"cba"
    report = {"protocol": version, "caps": caps}
    if caps & urpc.CAP_LIVE_QUEUES:
        lanes = [ch.add_queue() for _ in range(3)]            # three more queue pairs, while calls are running
        for i in range(a.calls):
            ok &= ch.call(1, b"%d" % i) == (b"%d" % i)[::-1]  # spread over the four lanes in turn
        report["sent_per_lane"] = [s for s, _ in ch.queue_stats()]
        ch.remove_queue(lanes[1])                             # waits for the calls in flight on that lane
        ok &= ch.call(1, b"after") == b"retfa" and len(ch.queues) == 2
    if caps & urpc.CAP_ACK:
        ch.call_async(7, b"job", user_ctx=42, want_ack=True)  # the server acknowledges, then answers
        events, deadline = [], time.monotonic() + 5
        while len(events) < 2 and time.monotonic() < deadline:
            events += ch.poll()
        report["events"] = [(e[0], e[1]) for e in events]
        ok &= report["events"] == [(urpc.POLL_ACK, 42), (urpc.POLL_RSP, 42)] and events[1][3] == b"deferred:job"
    urpc.async_events()
    srv.register(2, lambda b: b)                              # attached clients hear about it
    deadline = time.monotonic() + 5
    heard = False
    while caps and not heard and time.monotonic() < deadline:
        heard = any(t == urpc.EVENT_FUNC_CHANGED for t, _, _ in urpc.async_events())
        time.sleep(0.002)
    ok &= heard or not caps
    report["tasks"] = {k: v for k, v in urpc.ctl_stats().items() if k.startswith("tasks_")}
    ch.close()
    srv.stop()
    urpc.uninit()
    report["ok"] = bool(ok)
    print(json.dumps(report))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
