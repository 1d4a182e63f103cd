#!/usr/bin/env python
"""UMQ sample: two queues bound to each other exchange messages (bind-info exchange, buffer allocation, enqueue /
dequeue, credits flowing back), then print the queue statistics. Counterpart of the reference's umq example
(src/urpc/examples/umq).

    python examples/umq_pingpong.py [--rounds N] [--size BYTES]
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from umdk_b200 import umq  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rounds", type=int, default=500)
    ap.add_argument("--size", type=int, default=1024)
    a = ap.parse_args()
    umq.init(flow_control=True)
    left, right = umq.Queue("left", depth=32), umq.Queue("right", depth=32)
    left.bind(right.bind_info())
    right.bind(left.bind_info())
    payload = bytes(i & 0xff for i in range(a.size))
    ok = True
    t0 = time.perf_counter()
    for i in range(a.rounds):
        left.send(payload)
        ok &= right.recv() == payload
        right.send(payload[::-1])
        ok &= left.recv() == payload[::-1]
    dt = time.perf_counter() - t0
    out = {"ok": bool(ok), "round_trip_us": round(dt / a.rounds * 1e6, 1), "left": left.io_stats(),
           "flow_control": right.flow_control_stats()}
    left.close()
    right.close()
    umq.uninit()
    print(json.dumps(out))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
