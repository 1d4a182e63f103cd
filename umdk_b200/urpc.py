"""Python binding of URPC, remote procedure calls over UMQ / URMA (csrc/urpc: liburpc).

One process can serve functions (``serve`` + ``Server.register``; a polling thread executes them) and call them
through a ``Channel`` (``call`` synchronously, or ``call_async`` + ``poll``). Follows the reference's framework
API (urpc_func_call / urpc_func_poll / urpc_func_return, keepalive callback, request timeouts;
src/urpc/include/framework/urpc_framework_api.h).
"""
from __future__ import annotations

import ctypes
import os
import threading
import time
from typing import Callable, Dict, List, Optional, Tuple

from . import _native

ERR_TIMEOUT, ERR_SESSION_CLOSE, ERR_FUNC_NOT_FOUND = -110, -104, -38
POLL_REQ, POLL_RSP, POLL_ERR, POLL_TIMEOUT = 1, 2, 3, 4


class UrpcError(RuntimeError):
    def __init__(self, what: str, code: int):
        super().__init__(f"{what}: {code}")
        self.code = code


class _Config(ctypes.Structure):
    _fields_ = [("role", ctypes.c_int), ("dev_name", ctypes.c_char * 64), ("keepalive_interval_ms", ctypes.c_uint32),
                ("keepalive_miss_limit", ctypes.c_uint32), ("default_timeout_ms", ctypes.c_uint32)]


class _Sge(ctypes.Structure):
    _fields_ = [("addr", ctypes.c_void_p), ("len", ctypes.c_uint32)]


class _CallWr(ctypes.Structure):
    _fields_ = [("func_id", ctypes.c_uint64), ("args", ctypes.POINTER(_Sge)), ("num_args", ctypes.c_uint32),
                ("user_ctx", ctypes.c_uint64)]


class _CallOpt(ctypes.Structure):
    _fields_ = [("timeout_ms", ctypes.c_uint32), ("sync", ctypes.c_int), ("rsp_buf", ctypes.c_void_p),
                ("rsp_buf_len", ctypes.c_uint32), ("rsp_len", ctypes.POINTER(ctypes.c_uint32)),
                ("want_ack", ctypes.c_int)]


class _ChannelCfg(ctypes.Structure):
    _fields_ = [("timeout_ms", ctypes.c_uint32), ("attached", ctypes.c_int), ("lost", ctypes.c_int),
                ("sealed", ctypes.c_int), ("proto_version", ctypes.c_int), ("proto_caps", ctypes.c_uint32),
                ("pending_calls", ctypes.c_uint32), ("server_ip", ctypes.c_char * 64),
                ("server_port", ctypes.c_uint16)]


class _CtlStats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in ("tasks_started", "tasks_done", "tasks_failed", "tasks_timed_out",
                                               "notices_sent", "sessions_retired")] + \
               [("tasks_live", ctypes.c_uint32), ("timers_armed", ctypes.c_uint32)]


class _AsyncEvent(ctypes.Structure):
    _fields_ = [("type", ctypes.c_int), ("chid", ctypes.c_uint32), ("detail", ctypes.c_int)]


POLL_REQ, POLL_RSP, POLL_ERR, POLL_TIMEOUT, POLL_ACK = 1, 2, 3, 4, 5
EVENT_CHANNEL_LOST, EVENT_CHANNEL_REFRESHED, EVENT_FUNC_CHANGED = 1, 2, 3
CAP_LIVE_QUEUES, CAP_ACK, CAP_TASK_CANCEL = 1, 2, 4
ERR_VERSION, ERR_CANCELED = -71, -125


class _PollMsg(ctypes.Structure):
    _fields_ = [("event", ctypes.c_int), ("func_id", ctypes.c_uint64), ("req_id", ctypes.c_uint32),
                ("user_ctx", ctypes.c_uint64), ("data", ctypes.c_void_p), ("len", ctypes.c_uint32),
                ("status", ctypes.c_int), ("priv", ctypes.c_void_p)]


class _Stats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in ("calls", "responses", "timeouts", "errors", "requests_served",
                                               "keepalive_sent", "keepalive_lost", "bytes_tx", "bytes_rx")]


_FUNC = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p,
                         ctypes.POINTER(ctypes.c_uint32), ctypes.c_void_p)
_KA_CB = ctypes.CFUNCTYPE(None, ctypes.c_uint32, ctypes.c_int, ctypes.c_void_p)

_lib_cache = None
_keep: List[object] = []   # ctypes callbacks must outlive their registration


def _lib():
    global _lib_cache
    if _lib_cache is None:
        _lib_cache = ctypes.CDLL(os.path.join(_native.lib_dir(), "libumdk_urpc.so"))
    return _lib_cache


def init(dev: str = "shm0", keepalive_interval_ms: int = 0, keepalive_miss_limit: int = 3,
         default_timeout_ms: int = 5000) -> None:
    cfg = _Config()
    cfg.role, cfg.dev_name = 2, dev.encode()
    cfg.keepalive_interval_ms, cfg.keepalive_miss_limit = keepalive_interval_ms, keepalive_miss_limit
    cfg.default_timeout_ms = default_timeout_ms
    rc = _lib().urpc_init(ctypes.byref(cfg))
    if rc != 0:
        raise UrpcError("urpc_init", rc)


def set_psk(key_hex: str = "", identity: str = "") -> None:
    """Pre-shared key for servers started and channels attached afterwards: the connection handshake runs in TLS 1.3
    PSK and every payload is sealed with AES-256-GCM. An empty key switches both off."""
    rc = _lib().urpc_set_psk(key_hex.encode(), identity.encode())
    if rc != 0:
        raise UrpcError("urpc_set_psk", rc)


def set_tls_files(ca_file: str = "", cert_file: str = "", key_file: str = "") -> None:
    """Certificates instead of a shared key: the connection handshake runs in TLS 1.3 with mutual authentication
    against ``ca_file``. Three empty strings switch it off."""
    rc = _lib().urpc_set_tls_files(ca_file.encode(), cert_file.encode(), key_file.encode())
    if rc != 0:
        raise UrpcError("urpc_set_tls_files", rc)


PERF_POINTS = ("func_call", "call_to_response", "func_exec", "func_return")
_REC_CB = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p)
_LOG_CB = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_char_p)


def perf_recorder(cb: Optional[Callable[[str, int], None]]) -> None:
    """cb(point name, nanoseconds) at every record point (see PERF_POINTS); None unregisters."""
    if cb is None:
        _lib().urpc_perf_recorder_register(None, None)
        return
    c = _REC_CB(lambda pt, ns, _ctx: cb(PERF_POINTS[pt] if 0 <= pt < len(PERF_POINTS) else str(pt), int(ns)))
    _keep.append(c)
    _lib().urpc_perf_recorder_register(c, None)


def log_config(level: int, cb: Optional[Callable[[int, str], None]] = None) -> None:
    """Log level 0 (errors) .. 4 (debug); cb(level, message) replaces the stderr sink."""
    c = None
    if cb is not None:
        c = _LOG_CB(lambda lvl, msg: cb(int(lvl), msg.decode(errors="replace")))
        _keep.append(c)
    rc = _lib().urpc_log_config_set(level, c)
    if rc != 0:
        raise UrpcError("urpc_log_config_set", rc)


class _MemRef(ctypes.Structure):
    _fields_ = [("mem_h", ctypes.c_uint64), ("addr", ctypes.c_uint64), ("len", ctypes.c_uint32)]


def register_memory(addr: int, nbytes: int) -> int:
    """Registers memory whose address can then be passed by reference with ``Channel.call_ref``."""
    lib = _lib()
    lib.urpc_mem_seg_register.restype = ctypes.c_uint64
    h = lib.urpc_mem_seg_register(ctypes.c_void_p(addr), ctypes.c_uint64(nbytes))
    if not h:
        raise UrpcError("urpc_mem_seg_register", -1)
    return int(h)


def unregister_memory(mem_h: int) -> None:
    _lib().urpc_mem_seg_unregister(ctypes.c_uint64(mem_h))


def ref_count() -> int:
    """Inside a handler: how many by-reference arguments the request being handled carries."""
    return int(_lib().urpc_ref_count(None))


def ref_read(idx: int, offset: int = 0, nbytes: Optional[int] = None) -> bytes:
    """Inside a handler: pulls bytes of by-reference argument ``idx`` from the caller's memory."""
    lib = _lib()
    if nbytes is None:
        n = ctypes.c_uint32(0)
        if lib.urpc_ref_len(None, idx, ctypes.byref(n)) != 0:
            raise UrpcError("urpc_ref_len", -22)
        nbytes = n.value - offset
    buf = ctypes.create_string_buffer(nbytes)
    rc = lib.urpc_ref_read(None, idx, ctypes.c_uint64(offset), buf, nbytes)
    if rc != 0:
        raise UrpcError("urpc_ref_read", rc)
    return buf.raw


def admin_query(command: str) -> str:
    """The management report (`version`, `stats`, `perf`, `channels`, `sessions`, `functions`) as text."""
    buf = ctypes.create_string_buffer(16384)
    n = _lib().urpc_admin_query(command.encode(), buf, len(buf))
    return buf.value.decode() if n >= 0 else ""


def uninit() -> None:
    _lib().urpc_uninit()
    _keep.clear()


def stats() -> dict:
    s = _Stats()
    _lib().urpc_stats_get(ctypes.byref(s))
    return {n: int(getattr(s, n)) for n, _ in _Stats._fields_}


def ctl_stats() -> dict:
    """Counters of the server's control-plane task engine (tasks started / done / failed, notices, live tasks)."""
    st = _CtlStats()
    _lib().urpc_ctl_stats_get(ctypes.byref(st))
    return {n: int(getattr(st, n)) for n, _ in _CtlStats._fields_}


def async_events(max_n: int = 32) -> List[Tuple[int, int, int]]:
    """[(event type, channel id, detail)]: lost channels, refreshed channels, function-table changes."""
    ev = (_AsyncEvent * max_n)()
    n = _lib().urpc_async_event_get(ev, max_n)
    return [(ev[i].type, int(ev[i].chid), ev[i].detail) for i in range(max(n, 0))]


def on_keepalive(cb: Callable[[int, bool], None]) -> None:
    """cb(channel_id, alive) when a peer stops or resumes answering keepalive probes."""
    c = _KA_CB(lambda chid, alive, _ctx: cb(int(chid), bool(alive)))
    _keep.append(c)
    _lib().urpc_keepalive_callback_register(c, None)


class Server:
    """Serves registered functions from background polling threads. With ``threads`` > 1 each thread serves its share
    of the attached clients (``urpc_server_poll_shard``: session number modulo the thread count)."""

    def __init__(self, ip: str = "127.0.0.1", port: int = 0, threads: int = 1):
        p = _lib().urpc_server_start(ip.encode(), port)
        if p <= 0:
            raise UrpcError("urpc_server_start", p)
        self.ip, self.port = ip, p
        self._stop = threading.Event()
        self.paused = False   # True: requests are left unanswered (to exercise timeouts / keepalive)
        # requests of functions without a registered handler reach `deferred(func_id, args)`; it returns the answer
        # bytes, or (answer, status), or None to leave the request unanswered; it runs after `defer_s` seconds
        self.deferred: Optional[Callable[[int, bytes], object]] = None
        self.defer_s = 0.0
        self.return_codes: List[int] = []   # urpc_func_return results of deferred answers
        self.threads = max(1, int(threads))
        self.served_by: List[int] = [0] * self.threads   # requests handed to `deferred`, per polling thread
        self._thrs = [threading.Thread(target=self._loop, args=(k,), daemon=True) for k in range(self.threads)]
        for t in self._thrs:
            t.start()

    def register(self, func_id: int, fn: Callable[[bytes], bytes]) -> None:
        def handler(args, n, rsp, rsp_len, _ctx):
            try:
                out = fn(ctypes.string_at(args, n) if n else b"")
            except Exception:
                return -1
            if len(out) > rsp_len[0]:
                return -1
            ctypes.memmove(rsp, out, len(out))
            rsp_len[0] = len(out)
            return 0
        c = _FUNC(handler)
        _keep.append(c)
        rc = _lib().urpc_func_register(ctypes.c_uint64(func_id), c, None)
        if rc != 0:
            raise UrpcError("urpc_func_register", rc)

    def _loop(self, shard: int = 0):
        msgs = (_PollMsg * 16)()
        lib = _lib()
        while not self._stop.is_set():
            if self.paused:
                time.sleep(0.005)
                continue
            n = lib.urpc_server_poll_shard(shard, self.threads, msgs, 16)
            for i in range(max(n, 0)):
                m = msgs[i]
                if self.deferred is not None and m.event == POLL_REQ:   # registered functions ran inside the library
                    self.served_by[shard] += 1
                    args = ctypes.string_at(m.data, m.len) if m.data and m.len else b""
                    if self.defer_s:
                        time.sleep(self.defer_s)
                    out = self.deferred(int(m.func_id), args)
                    if out is not None:
                        body, status = out if isinstance(out, tuple) else (out, 0)
                        self.return_codes.append(lib.urpc_func_return(ctypes.byref(m), body, len(body), status))
                lib.urpc_msg_release(ctypes.byref(m))
            if n <= 0:
                time.sleep(0.0002)

    def stop(self):
        self._stop.set()
        for t in self._thrs:
            t.join(timeout=2)


class Channel:
    """A client channel attached to one server. ``queues`` > 1 gives it that many queue pairs (made with
    ``urpc_queue_create`` and added before the attach): calls then spread over them in turn, or go to the one
    ``call(..., queue=i)`` names, and each response returns on the queue pair of its request."""

    def __init__(self, ip: str, port: int, queues: int = 1):
        lib = _lib()
        ch = lib.urpc_channel_create()
        if ch < 0:
            raise UrpcError("urpc_channel_create", ch)
        self.id = ch
        self.queues: List[int] = []
        lib.urpc_queue_create.restype = ctypes.c_uint64
        rc = 0
        for _ in range(queues if queues > 1 else 0):
            q = lib.urpc_queue_create(None)
            rc = lib.urpc_channel_queue_add(ch, ctypes.c_uint64(q)) if q else -1
            if q:
                self.queues.append(q)
            if rc != 0:
                break
        if rc == 0:
            rc = lib.urpc_channel_server_attach(ch, ip.encode(), port)
        if rc != 0:
            lib.urpc_channel_destroy(ch)
            for q in self.queues:
                lib.urpc_queue_destroy(ctypes.c_uint64(q))
            raise UrpcError("urpc_channel_server_attach", rc)

    def _call(self, wr, opt, queue: Optional[int]):
        if queue is None:
            return _lib().urpc_func_call(self.id, ctypes.byref(wr), ctypes.byref(opt))
        return _lib().urpc_func_call_on(self.id, ctypes.c_uint64(self.queues[queue]), ctypes.byref(wr),
                                        ctypes.byref(opt))

    def queue_stats(self) -> List[Tuple[int, int]]:
        """(messages sent, messages received) of every explicit queue pair, in lane order."""
        out = []
        for q in self.queues:
            st = (ctypes.c_uint64 * 4)()
            _lib().urpc_queue_stats_get(ctypes.c_uint64(q), st, 4)
            out.append((int(st[0]), int(st[2])))
        return out

    def _wr(self, func_id: int, args: bytes, user_ctx: int):
        buf = ctypes.create_string_buffer(args, len(args)) if args else None
        sge = _Sge(ctypes.cast(buf, ctypes.c_void_p) if buf else None, len(args))
        wr = _CallWr(func_id, ctypes.pointer(sge), 1 if args else 0, user_ctx)
        return wr, (buf, sge)

    def call(self, func_id: int, args: bytes = b"", timeout_ms: int = 0, max_rsp: int = 65536,
             queue: Optional[int] = None) -> bytes:
        wr, keep = self._wr(func_id, args, 0)
        rsp = ctypes.create_string_buffer(max_rsp)
        n = ctypes.c_uint32(0)
        opt = _CallOpt(timeout_ms, 1, ctypes.cast(rsp, ctypes.c_void_p), max_rsp, ctypes.pointer(n), 0)
        rc = self._call(wr, opt, queue)
        if rc != 0:
            raise UrpcError("urpc_func_call", rc)
        return rsp.raw[:n.value]

    def call_ref(self, func_id: int, args: bytes, refs: List[Tuple[int, int, int]], timeout_ms: int = 0,
                 max_rsp: int = 65536) -> bytes:
        """Call with arguments by reference: ``refs`` = [(memory handle from register_memory, address, length)];
        the server pulls what it needs with ``ref_read`` instead of receiving the bytes inline."""
        wr, keep = self._wr(func_id, args, 0)
        arr = (_MemRef * len(refs))(*[_MemRef(h, a, n) for h, a, n in refs])
        rsp = ctypes.create_string_buffer(max_rsp)
        n = ctypes.c_uint32(0)
        opt = _CallOpt(timeout_ms, 1, ctypes.cast(rsp, ctypes.c_void_p), max_rsp, ctypes.pointer(n), 0)
        rc = _lib().urpc_func_call_ref(self.id, ctypes.byref(wr), arr, len(refs), ctypes.byref(opt))
        if rc != 0:
            raise UrpcError("urpc_func_call_ref", rc)
        return rsp.raw[:n.value]

    def add_queue(self) -> int:
        """Adds one more queue pair to the channel, attached or not (an attached channel needs a server that
        negotiated protocol version 2). -> index for ``call(..., queue=i)``."""
        lib = _lib()
        lib.urpc_queue_create.restype = ctypes.c_uint64
        q = lib.urpc_queue_create(None)
        if not q:
            raise UrpcError("urpc_queue_create", -1)
        rc = lib.urpc_channel_queue_add(self.id, ctypes.c_uint64(q))
        if rc != 0:
            lib.urpc_queue_destroy(ctypes.c_uint64(q))
            raise UrpcError("urpc_channel_queue_add", rc)
        self.queues.append(q)
        return len(self.queues) - 1

    def remove_queue(self, index: int) -> None:
        """Takes a queue pair out of the channel (waits for the calls in flight on it) and destroys the queue."""
        q = self.queues[index]
        rc = _lib().urpc_channel_queue_rm(self.id, ctypes.c_uint64(q))
        if rc != 0:
            raise UrpcError("urpc_channel_queue_rm", rc)
        self.queues.pop(index)
        _lib().urpc_queue_destroy(ctypes.c_uint64(q))

    def protocol(self) -> Tuple[int, int]:
        """(negotiated protocol version, capability bits) of the attach; (0, 0) while detached."""
        cfg = _ChannelCfg()
        _lib().urpc_channel_cfg_get(self.id, ctypes.byref(cfg))
        return cfg.proto_version, cfg.proto_caps

    def cancel(self, req_id: int) -> None:
        rc = _lib().urpc_channel_task_cancel(self.id, req_id)
        if rc != 0:
            raise UrpcError("urpc_channel_task_cancel", rc)

    def call_async(self, func_id: int, args: bytes = b"", user_ctx: int = 0, timeout_ms: int = 0,
                   queue: Optional[int] = None, want_ack: bool = False) -> int:
        wr, keep = self._wr(func_id, args, user_ctx)
        opt = _CallOpt(timeout_ms, 0, None, 0, None, int(want_ack))
        rc = self._call(wr, opt, queue)
        if rc < 0:
            raise UrpcError("urpc_func_call", rc)
        return rc   # request id

    def poll(self, max_n: int = 16) -> List[Tuple[int, int, int, bytes]]:
        """[(event, user_ctx, status, payload)] for completed asynchronous calls."""
        msgs = (_PollMsg * max_n)()
        n = _lib().urpc_func_poll(self.id, msgs, max_n)
        out = []
        for i in range(max(n, 0)):
            m = msgs[i]
            out.append((m.event, int(m.user_ctx), m.status, ctypes.string_at(m.data, m.len) if m.data and m.len else b""))
            _lib().urpc_msg_release(ctypes.byref(m))
        return out

    def close(self):
        if self.id >= 0:
            _lib().urpc_channel_server_detach(self.id)
            _lib().urpc_channel_destroy(self.id)
            for q in self.queues:
                _lib().urpc_queue_destroy(ctypes.c_uint64(q))
            self.queues = []
            self.id = -1
