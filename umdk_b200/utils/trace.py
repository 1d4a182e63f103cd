"""NVTX ranges around the framework's operator calls, so that a timeline tool shows `umdk.dispatch`, `umdk.combine`,
`umdk.moe_fused` ... next to the kernels they launch. Off by default (the push / pop pair costs a few hundred
nanoseconds per call); switch on with `enable()` or `UMDK_NVTX=1`. The reference's counterpart is the profiler trace
filtered by kernel name in its example utilities (src/cam/examples/utils.py:163-232)."""
from __future__ import annotations

import contextlib
import functools
import os

import torch

_enabled = os.environ.get("UMDK_NVTX", "0") not in ("", "0")
_calls = {}


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


def call_counts() -> dict:
    """How often each traced operator ran while tracing was on (works without a GPU; used by the tests)."""
    return dict(_calls)


@contextlib.contextmanager
def range(name: str):
    if not _enabled:
        yield
        return
    _calls[name] = _calls.get(name, 0) + 1
    on_gpu = torch.cuda.is_available()
    if on_gpu:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on_gpu:
            torch.cuda.nvtx.range_pop()


def traced(name: str):
    """Decorator form of `range`."""
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **kw):
            if not _enabled:
                return fn(*a, **kw)
            with range(name):
                return fn(*a, **kw)
        return wrapper
    return deco
