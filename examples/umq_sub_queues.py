#!/usr/bin/env python
"""UMQ sample: many connections on few resources. Two main queues own the receive buffers and the jetties; every
connection is a pair of sub queues that receive through its main queue's shared buffers and send through an endpoint
borrowed from the jetty pool. A message beyond the receive buffer size is pulled by the receiver from the sender's
memory. Counterpart of the reference's shared-JFR / jetty-pool mode of its UB transport.

    python examples/umq_sub_queues.py [--connections N]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from umdk_b200 import umq  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--connections", type=int, default=32)
    a = ap.parse_args()
    umq.init(flow_control=True)
    side_a = umq.Queue("side-a", depth=128, main=True, share_transport=True)
    side_b = umq.Queue("side-b", depth=128, main=True, share_transport=True)
    conns = []
    for i in range(a.connections):
        x, y = umq.Queue(f"a{i}", depth=8, sub_of=side_a), umq.Queue(f"b{i}", depth=8, sub_of=side_b)
        x.bind(y.bind_info())
        y.bind(x.bind_info())
        conns.append((x, y))
    ok = True
    for rnd in range(5):
        for i, (x, y) in enumerate(conns):
            x.send(b"request %d.%d" % (i, rnd))
        for i, (x, y) in enumerate(conns):
            ok &= y.recv() == b"request %d.%d" % (i, rnd)
            y.send(b"reply %d.%d" % (i, rnd))
        for i, (x, y) in enumerate(conns):
            ok &= x.recv() == b"reply %d.%d" % (i, rnd)
    big = os.urandom(1 << 20)                      # 128 receive buffers' worth: travels as a descriptor and is pulled
    conns[0][0].send(big)
    ok &= conns[0][1].recv() == big
    pool = umq.jetty_pool_stats()
    pulled = conns[0][1].io_stats()["pull_rx"]
    for x, y in conns:
        x.close()
        y.close()
    side_a.close()
    side_b.close()
    umq.uninit()
    ok &= pool["total_num"] == 2 and pool["sub_queues"] == 2 * a.connections and pulled == 1
    print(json.dumps({"ok": bool(ok), "connections": a.connections, "jetties": pool["total_num"],
                      "borrowed_posts": pool["acc_alloc_num"], "misses": pool["acc_miss_num"], "pulled_messages": pulled}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
