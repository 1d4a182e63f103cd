"""Python binding of UMQ, the message queue over URMA (csrc/umq: libumdk_umq.so).

``init()`` once per process, then ``Queue`` objects that exchange bind information with a peer queue and move byte
messages (``send`` / ``recv``) through pooled buffers with credit-based flow control. Mirrors the reference's base
API (``umq_enqueue`` / ``umq_dequeue``; doc/en/urpc/UMQ API Guide) at message granularity.
"""
from __future__ import annotations

import ctypes
import os
import time
from typing import Optional

from . import _native

FEATURE_API_BASE, FEATURE_API_PRO, FEATURE_STATS, FEATURE_PERF, FEATURE_FLOW_CONTROL = 0x1, 0x2, 0x8, 0x10, 0x20
BIND_INFO_SIZE = 128
ERR_EAGAIN = -11


class UmqError(RuntimeError):
    pass


class _InitCfg(ctypes.Structure):
    _fields_ = [("feature", ctypes.c_uint32), ("trans_mode", ctypes.c_int), ("dev_name", ctypes.c_char * 64),
                ("block_size_kb", ctypes.c_uint32), ("pool_bytes", ctypes.c_uint64)]


TRANS_MODE_UB, TRANS_MODE_IPC = 0, 3   # umq_trans_mode_t


class _CreateOpt(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 32), ("rx_buf_size", ctypes.c_uint32), ("tx_buf_size", ctypes.c_uint32),
                ("rx_depth", ctypes.c_uint32), ("tx_depth", ctypes.c_uint32), ("mode", ctypes.c_int),
                ("token", ctypes.c_uint32), ("transport", ctypes.c_uint32), ("create_flag", ctypes.c_uint32),
                ("share_rq_umqh", ctypes.c_uint64)]


class _JettyPoolStats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in
                ("total_num", "err_num", "acc_alloc_num", "acc_free_num", "acc_miss_num", "sub_queues")]


CREATE_FLAG_MAIN, CREATE_FLAG_SHARE_TRANSPORT, CREATE_FLAG_SUB = 1, 2, 4


def jetty_pool_stats() -> dict:
    st = _JettyPoolStats()
    _lib().umq_jetty_pool_stats_get(ctypes.byref(st))
    return {n: int(getattr(st, n)) for n, _ in _JettyPoolStats._fields_}


class _Buf(ctypes.Structure):
    pass


_Buf._fields_ = [("qbuf_next", ctypes.POINTER(_Buf)), ("umqh", ctypes.c_uint64),
                 ("total_data_size", ctypes.c_uint32), ("buf_size", ctypes.c_uint32), ("data_size", ctypes.c_uint32),
                 ("headroom_size", ctypes.c_uint16), ("status", ctypes.c_uint16), ("user_ctx", ctypes.c_uint64),
                 ("buf_data", ctypes.c_void_p), ("rsvd", ctypes.c_uint64 * 8)]


class _IoStats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in
                ("tx_msgs", "tx_bytes", "rx_msgs", "rx_bytes", "tx_errors", "rx_errors", "tx_eagain", "pull_tx",
                 "pull_rx")]


class _FcStats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in
                ("credits_local", "credits_remote", "credits_granted", "credits_returned", "stalls", "window")]


_lib_cache = None


def _lib():
    global _lib_cache
    if _lib_cache is None:
        lib = ctypes.CDLL(os.path.join(_native.lib_dir(), "libumdk_umq.so"))
        lib.umq_create.restype = ctypes.c_uint64
        lib.umq_buf_alloc.restype = ctypes.POINTER(_Buf)
        lib.umq_buf_alloc.argtypes = [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint64]
        lib.umq_dequeue.restype = ctypes.POINTER(_Buf)
        lib.umq_dequeue.argtypes = [ctypes.c_uint64]
        lib.umq_enqueue.argtypes = [ctypes.c_uint64, ctypes.POINTER(_Buf), ctypes.POINTER(ctypes.POINTER(_Buf))]
        lib.umq_buf_free.argtypes = [ctypes.POINTER(_Buf)]
        lib.umq_bind_info_get.restype = ctypes.c_uint32
        for f in (lib.umq_destroy, lib.umq_unbind, lib.umq_state_get):
            f.argtypes = [ctypes.c_uint64]
        lib.umq_bind.argtypes = [ctypes.c_uint64, ctypes.c_char_p, ctypes.c_uint32]
        lib.umq_bind_info_get.argtypes = [ctypes.c_uint64, ctypes.c_char_p, ctypes.c_uint32]
        lib.umq_stats_io_get.argtypes = [ctypes.c_uint64, ctypes.POINTER(_IoStats)]
        lib.umq_stats_flow_control_get.argtypes = [ctypes.c_uint64, ctypes.POINTER(_FcStats)]
        _lib_cache = lib
    return _lib_cache


def init(dev: str = "shm0", flow_control: bool = True, block_size_kb: int = 8, pool_bytes: int = 0) -> None:
    cfg = _InitCfg()
    cfg.feature = FEATURE_API_BASE | FEATURE_STATS | (FEATURE_FLOW_CONTROL if flow_control else 0)
    cfg.dev_name, cfg.block_size_kb, cfg.pool_bytes = dev.encode(), block_size_kb, pool_bytes
    if _lib().umq_init(ctypes.byref(cfg)) != 0:
        raise UmqError("umq_init failed")


def uninit() -> None:
    _lib().umq_uninit()


PERF_RECORDS = ("enqueue", "dequeue", "post_tx", "poll_rx", "buf_alloc")
_PERF_CB = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p)
_LOG_CB = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_char_p)
_keep = []   # ctypes callbacks must outlive their registration


class _AsyncEvent(ctypes.Structure):
    _fields_ = [("type", ctypes.c_int), ("umqh", ctypes.c_uint64), ("detail", ctypes.c_int)]


def io_perf_callback(cb) -> None:
    """cb(record name, nanoseconds) after every queue operation; None unregisters."""
    if cb is None:
        _lib().umq_io_perf_callback_register(None, None)
        return
    c = _PERF_CB(lambda rec, ns, _ctx: cb(PERF_RECORDS[rec] if 0 <= rec < len(PERF_RECORDS) else str(rec), int(ns)))
    _keep.append(c)
    _lib().umq_io_perf_callback_register(c, None)


def log_config(level: int, cb=None) -> None:
    """Log level 0 (errors) .. 4 (debug); cb(level, message) replaces the stderr sink."""
    c = None
    if cb is not None:
        c = _LOG_CB(lambda lvl, msg: cb(int(lvl), msg.decode(errors="replace")))
        _keep.append(c)
    rc = _lib().umq_log_config_set(level, c)
    if rc != 0:
        raise UmqError(f"umq_log_config_set failed: {rc}")


def async_events() -> list:
    """Drains the asynchronous event queue: [(type, queue handle, detail)]; type 1 = queue entered the error state."""
    out = []
    ev = _AsyncEvent()
    while _lib().umq_async_event_get(ctypes.byref(ev)) == 0:
        out.append((int(ev.type), int(ev.umqh), int(ev.detail)))
    return out


def trace_start(path: str, flush_interval_ms: int = 100, ring_entries: int = 4096) -> None:
    """Starts writing one line `start_ns tid record duration_ns` per queue operation to `path` (per-thread rings
    drained by a timer thread)."""
    rc = _lib().umq_trace_start(path.encode(), flush_interval_ms, ring_entries)
    if rc != 0:
        raise UmqError(f"umq_trace_start failed: {rc}")


def trace_stop() -> dict:
    """Stops the trace, flushes what is left and returns {"written", "dropped"}."""
    lib = _lib()
    rc = lib.umq_trace_stop()
    if rc != 0:
        raise UmqError(f"umq_trace_stop failed: {rc}")
    w, d = ctypes.c_uint64(), ctypes.c_uint64()
    lib.umq_trace_stats(ctypes.byref(w), ctypes.byref(d))
    return {"written": int(w.value), "dropped": int(d.value)}


class Queue:
    def __init__(self, name: str, depth: int = 128, buf_size: int = 0, token: int = 0x756d71,
                 transport: Optional[int] = None, main: bool = False, share_transport: bool = False,
                 sub_of: Optional["Queue"] = None):
        """``transport``: a transport mode for this queue (TRANS_MODE_UB = URMA, TRANS_MODE_IPC = the in-process
        transport, or a mode registered with umq_transport_register); None = the mode given to ``init``.
        ``main``: the queue can host sub queues (``share_transport``: its endpoint also joins the jetty pool);
        ``sub_of``: make a sub queue of that main queue (no endpoint and no receive buffers of its own)."""
        o = _CreateOpt()
        o.create_flag = (CREATE_FLAG_MAIN if main else 0) | (CREATE_FLAG_SHARE_TRANSPORT if share_transport else 0) | \
            (CREATE_FLAG_SUB if sub_of is not None else 0)
        o.share_rq_umqh = sub_of.h if sub_of is not None else 0
        o.name, o.rx_depth, o.tx_depth, o.rx_buf_size, o.tx_buf_size, o.token = \
            name.encode(), depth, depth, buf_size, buf_size, token
        o.transport = 0 if transport is None else transport + 1
        self.h = _lib().umq_create(ctypes.byref(o))
        if not self.h:
            raise UmqError("umq_create failed")

    def bind_info(self) -> bytes:
        buf = ctypes.create_string_buffer(BIND_INFO_SIZE)
        n = _lib().umq_bind_info_get(self.h, buf, BIND_INFO_SIZE)
        if n == 0:
            raise UmqError("umq_bind_info_get failed")
        return buf.raw[:n]

    def bind(self, peer_info: bytes) -> None:
        if _lib().umq_bind(self.h, peer_info, len(peer_info)) != 0:
            raise UmqError("umq_bind failed")

    def send(self, data: bytes, timeout_s: float = 5.0) -> None:
        lib = _lib()
        deadline = time.monotonic() + timeout_s
        while True:
            buf = lib.umq_buf_alloc(len(data), 1, self.h)
            if buf:
                break
            if time.monotonic() > deadline:
                raise UmqError("no buffer available")
            time.sleep(0.0005)
        b = buf.contents
        if b.buf_size < len(data):
            lib.umq_buf_free(buf)
            raise UmqError(f"message of {len(data)} bytes does not fit a {b.buf_size}-byte buffer")
        ctypes.memmove(b.buf_data, data, len(data))
        b.data_size = b.total_data_size = len(data)
        bad = ctypes.POINTER(_Buf)()
        while True:
            rc = lib.umq_enqueue(self.h, buf, ctypes.byref(bad))
            if rc == 0:
                return
            if rc != ERR_EAGAIN or time.monotonic() > deadline:
                lib.umq_buf_free(buf)
                raise UmqError(f"umq_enqueue failed: {rc}")
            self._progress()
            time.sleep(0.0002)

    def _progress(self):
        pass

    def recv(self, timeout_s: float = 5.0) -> Optional[bytes]:
        """Next message, or None when nothing arrives within the timeout."""
        lib = _lib()
        deadline = time.monotonic() + timeout_s
        while True:
            buf = lib.umq_dequeue(self.h)
            if buf:
                b = buf.contents
                data = ctypes.string_at(b.buf_data, b.data_size)
                lib.umq_buf_free(buf)
                return data
            if time.monotonic() > deadline:
                return None
            time.sleep(0.0002)

    def set_state(self, state: int) -> None:
        """0 = idle, 1 = ready, 2 = error (raises a queue-error event)."""
        if _lib().umq_state_set(self.h, state) != 0:
            raise UmqError("umq_state_set failed")

    def state(self) -> int:
        return int(_lib().umq_state_get(self.h))

    def io_stats(self) -> dict:
        s = _IoStats()
        _lib().umq_stats_io_get(self.h, ctypes.byref(s))
        return {n: int(getattr(s, n)) for n, _ in _IoStats._fields_}

    def flow_control_stats(self) -> dict:
        s = _FcStats()
        _lib().umq_stats_flow_control_get(self.h, ctypes.byref(s))
        return {n: int(getattr(s, n)) for n, _ in _FcStats._fields_}

    def close(self):
        if self.h:
            _lib().umq_unbind(self.h)
            _lib().umq_destroy(self.h)
            self.h = 0
