"""Operator ranges for timeline tools: off by default, counted per operator when switched on."""
import torch


def test_ranges_are_off_by_default_and_count_when_enabled():
    from umdk_b200 import Buffer
    from umdk_b200.utils import trace
    trace.enable(False)
    before = trace.call_counts().get("umdk.buffer.get_dispatch_layout", 0)
    buf = Buffer(None)
    idx = torch.randint(0, 8, (16, 2))
    buf.get_dispatch_layout(idx, 8)
    assert trace.call_counts().get("umdk.buffer.get_dispatch_layout", 0) == before
    trace.enable(True)
    try:
        buf.get_dispatch_layout(idx, 8)
        buf.get_dispatch_layout(idx, 8)
        with trace.range("user.section"):
            pass
    finally:
        trace.enable(False)
    counts = trace.call_counts()
    assert counts["umdk.buffer.get_dispatch_layout"] == before + 2 and counts["user.section"] >= 1
