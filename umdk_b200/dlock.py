"""Python binding of the distributed lock service (csrc/dlock: libumdk_dlock.so).

A ``Server`` owns the lock memory (ATOMIC / RW / FAIR locks with leases, 64-bit atomic objects); ``Client`` talks to
it over TCP for control operations and over URMA one-sided atomics for the lock words themselves. The C API follows
the reference's dlock client/server interface (src/ulock/dlock/lib/include/dlock_client_api.h, dlock_server_api.h).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence, Tuple

from . import _native

SUCCESS, EAGAIN, ALREADY_LOCKED, NOT_OWNER, TIMEOUT = 0, 0x1000, 0x1001, 0x1002, 0x1004
CLIENT_NOT_INIT, EASYNC, NO_ASYNC, ASYNC_AGAIN = 0x2000, 0x2004, 0x2005, 0x2006
BAD_RESPONSE, NOT_READY = 0x2001, 0x2002
ATOMIC, RW, FAIR = 0, 1, 2
EXCLUSIVE, SHARED = 0, 1


class DlockError(RuntimeError):
    def __init__(self, what: str, code: int):
        super().__init__(f"{what}: status 0x{code & 0xffffffff:x}")
        self.code = code


class _ServerCfg(ctypes.Structure):
    _fields_ = [("ip", ctypes.c_char * 32), ("port", ctypes.c_uint16), ("max_clients", ctypes.c_uint32),
                ("max_locks", ctypes.c_uint32), ("max_objects", ctypes.c_uint32),
                ("recovery_client_num", ctypes.c_uint32), ("recovery_timeout_ms", ctypes.c_uint32),
                ("dev_name", ctypes.c_char * 64)]


class _LockDesc(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 64), ("type", ctypes.c_int)]


class _LockReq(ctypes.Structure):
    _fields_ = [("lock_id", ctypes.c_int32), ("op", ctypes.c_int), ("expire_ms", ctypes.c_uint32)]


class _Stats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in
                ("trylock_ok", "trylock_busy", "unlock_ok", "unlock_fail", "extend_ok", "expired_takeover",
                 "heartbeat", "recovered_locks", "control_msgs", "data_msgs", "objects", "object_ops", "clients",
                 "tls_rejected", "sealed_rejected")]


_lib_cache = None


def _lib():
    global _lib_cache
    if _lib_cache is None:
        _lib_cache = ctypes.CDLL(os.path.join(_native.lib_dir(), "libumdk_dlock.so"))
    return _lib_cache


def _stats_dict(s: _Stats) -> dict:
    return {n: int(getattr(s, n)) for n, _ in _Stats._fields_}


def set_psk(key_hex: str = "", identity: str = "") -> None:
    """Pre-shared key for servers started and clients created afterwards: TLS 1.3 PSK on the control channel and
    AES-256-GCM sealed lock commands on the data channel. An empty key switches both off."""
    rc = _lib().dlock_set_psk(key_hex.encode(), identity.encode())
    if rc != 0:
        raise DlockError("set_psk", rc)


def set_tls_files(ca_file: str = "", cert_file: str = "", key_file: str = "") -> None:
    """Certificates instead of a shared key for servers started and clients created afterwards: the control channel
    runs TLS 1.3 with mutual authentication against ``ca_file``. Three empty strings switch it off."""
    rc = _lib().dlock_set_tls_files(ca_file.encode(), cert_file.encode(), key_file.encode())
    if rc != 0:
        raise DlockError("set_tls_files", rc)


class Server:
    def __init__(self, ip: str = "127.0.0.1", port: int = 0, dev: str = "shm0", recovery_clients: int = 0,
                 recovery_timeout_ms: int = 3000):
        cfg = _ServerCfg()
        cfg.ip, cfg.port, cfg.dev_name = ip.encode(), port, dev.encode()
        cfg.recovery_client_num, cfg.recovery_timeout_ms = recovery_clients, recovery_timeout_ms
        sid, p = ctypes.c_int(-1), ctypes.c_uint16(0)
        rc = _lib().dlock_server_start(ctypes.byref(cfg), ctypes.byref(sid), ctypes.byref(p))
        if rc != SUCCESS:
            raise DlockError("dlock_server_start", rc)
        self.id, self.ip, self.port = sid.value, ip, p.value

    def stats(self) -> dict:
        s = _Stats()
        _lib().dlock_get_server_debug_stats(self.id, ctypes.byref(s))
        return _stats_dict(s)

    def clear_stats(self) -> None:
        _lib().dlock_clear_server_debug_stats(self.id)

    def stop(self):
        if self.id >= 0:
            _lib().dlock_server_stop(self.id)
            self.id = -1


class Client:
    def __init__(self, ip: str, port: int):
        cid = ctypes.c_int(-1)
        rc = _lib().dlock_client_init(ctypes.byref(cid), ip.encode(), port)
        if rc != SUCCESS:
            raise DlockError("dlock_client_init", rc)
        self.id = cid.value

    def get_lock(self, name: str, kind: int = ATOMIC) -> int:
        d = _LockDesc()
        d.name, d.type = name.encode(), kind
        lid = ctypes.c_int32(-1)
        rc = _lib().dlock_get_lock(self.id, ctypes.byref(d), ctypes.byref(lid))
        if rc != SUCCESS:
            raise DlockError("dlock_get_lock", rc)
        return lid.value

    def trylock(self, lock_id: int, shared: bool = False, expire_ms: int = 10000) -> bool:
        """True if taken, False if somebody else holds it."""
        r = _LockReq(lock_id, SHARED if shared else EXCLUSIVE, expire_ms)
        rc = _lib().dlock_trylock(self.id, ctypes.byref(r))
        if rc == SUCCESS:
            return True
        if rc == EAGAIN:
            return False
        raise DlockError("dlock_trylock", rc)

    def lock(self, lock_id: int, shared: bool = False, expire_ms: int = 10000, timeout_ms: int = 5000) -> None:
        r = _LockReq(lock_id, SHARED if shared else EXCLUSIVE, expire_ms)
        rc = _lib().dlock_lock(self.id, ctypes.byref(r), timeout_ms)
        if rc != SUCCESS:
            raise DlockError("dlock_lock", rc)

    def unlock(self, lock_id: int) -> None:
        rc = _lib().dlock_unlock(self.id, lock_id)
        if rc != SUCCESS:
            raise DlockError("dlock_unlock", rc)

    def extend(self, lock_id: int, expire_ms: int) -> None:
        rc = _lib().dlock_lock_extend(self.id, lock_id, expire_ms)
        if rc != SUCCESS:
            raise DlockError("dlock_lock_extend", rc)

    def release_lock(self, lock_id: int) -> None:
        _lib().dlock_release_lock(self.id, lock_id)

    def batch_trylock(self, lock_ids: Sequence[int], expire_ms: int = 10000) -> List[int]:
        n = len(lock_ids)
        reqs = (_LockReq * n)(*[_LockReq(i, EXCLUSIVE, expire_ms) for i in lock_ids])
        res = (ctypes.c_int * n)()
        _lib().dlock_batch_trylock(self.id, n, reqs, res)
        return list(res)

    def batch_unlock(self, lock_ids: Sequence[int]) -> List[int]:
        n = len(lock_ids)
        ids = (ctypes.c_int32 * n)(*lock_ids)
        res = (ctypes.c_int * n)()
        _lib().dlock_batch_unlock(self.id, n, ids, res)
        return list(res)

    def heartbeat(self, timeout_ms: int = 1000) -> int:
        return _lib().dlock_client_heartbeat(self.id, timeout_ms)

    def reinit(self, ip: str, port: int) -> None:
        rc = _lib().dlock_client_reinit(self.id, ip.encode(), port)
        if rc != SUCCESS:
            raise DlockError("dlock_client_reinit", rc)

    def update_all_locks(self) -> None:
        rc = _lib().dlock_update_all_locks(self.id)
        if rc != SUCCESS:
            raise DlockError("dlock_update_all_locks", rc)

    def reinit_done(self) -> None:
        """After reinit + update_all_locks: tells the restarted server that this client is fully back."""
        rc = _lib().dlock_client_reinit_done(self.id)
        if rc != SUCCESS:
            raise DlockError("dlock_client_reinit_done", rc)

    def request_async(self, lock_id: int, op: int = EXCLUSIVE, expire_ms: int = 10000) -> None:
        """Sends a lock / unlock / extend request without waiting; collect the outcome with ``result()``."""
        r = _LockReq(lock_id, op, expire_ms)
        rc = _lib().dlock_lock_request_async(self.id, ctypes.byref(r))
        if rc != SUCCESS:
            raise DlockError("dlock_lock_request_async", rc)

    def result(self) -> Optional[int]:
        """Status of the outstanding asynchronous request, or None while the answer has not arrived."""
        res = ctypes.c_int(0)
        rc = _lib().dlock_lock_result_check(self.id, ctypes.byref(res))
        if rc == ASYNC_AGAIN:
            return None
        if rc in (NO_ASYNC, TIMEOUT, CLIENT_NOT_INIT):
            raise DlockError("dlock_lock_result_check", rc)
        return rc

    def batch_extend(self, lock_ids: Sequence[int], expire_ms: int) -> List[int]:
        n = len(lock_ids)
        reqs = (_LockReq * n)(*[_LockReq(i, 3, expire_ms) for i in lock_ids])
        res = (ctypes.c_int * n)()
        _lib().dlock_batch_lock_extend(self.id, n, reqs, res)
        return list(res)

    def batch_release(self, lock_ids: Sequence[int]) -> int:
        n = len(lock_ids)
        return _lib().dlock_batch_release_lock(self.id, n, (ctypes.c_int32 * n)(*lock_ids))

    def clear_stats(self) -> None:
        _lib().dlock_clear_client_debug_stats(self.id)

    # ---- 64-bit atomic objects ----
    def atomic_create(self, name: str, init: int = 0) -> int:
        oid = ctypes.c_int32(-1)
        rc = _lib().dlock_umo_atomic64_create(self.id, name.encode(), ctypes.c_uint64(init), ctypes.byref(oid))
        if rc != SUCCESS:
            raise DlockError("dlock_umo_atomic64_create", rc)
        return oid.value

    def atomic_get(self, name: str) -> int:
        oid = ctypes.c_int32(-1)
        rc = _lib().dlock_umo_atomic64_get(self.id, name.encode(), ctypes.byref(oid))
        if rc != SUCCESS:
            raise DlockError("dlock_umo_atomic64_get", rc)
        return oid.value

    def atomic_faa(self, obj_id: int, add: int) -> int:
        old = ctypes.c_uint64(0)
        rc = _lib().dlock_umo_atomic64_faa(self.id, obj_id, ctypes.c_uint64(add), ctypes.byref(old))
        if rc != SUCCESS:
            raise DlockError("dlock_umo_atomic64_faa", rc)
        return old.value

    def atomic_cas(self, obj_id: int, compare: int, swap: int) -> int:
        old = ctypes.c_uint64(0)
        rc = _lib().dlock_umo_atomic64_cas(self.id, obj_id, ctypes.c_uint64(compare), ctypes.c_uint64(swap),
                                           ctypes.byref(old))
        if rc != SUCCESS:
            raise DlockError("dlock_umo_atomic64_cas", rc)
        return old.value

    def atomic_snapshot(self, obj_id: int) -> int:
        v = ctypes.c_uint64(0)
        rc = _lib().dlock_umo_atomic64_get_snapshot(self.id, obj_id, ctypes.byref(v))
        if rc != SUCCESS:
            raise DlockError("dlock_umo_atomic64_get_snapshot", rc)
        return v.value

    def stats(self) -> dict:
        s = _Stats()
        _lib().dlock_get_client_debug_stats(self.id, ctypes.byref(s))
        return _stats_dict(s)

    def close(self):
        if self.id >= 0:
            _lib().dlock_client_deinit(self.id)
            self.id = -1
