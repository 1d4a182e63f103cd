"""KV-cache offload / prefetch manager (csrc/cam/kv_offload.cu): pinned host pool + cudaMemcpyAsync on a side stream."""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from .. import _native


def _iarr(v: Sequence[int]):
    return (ctypes.c_int * len(v))(*v)


class KvOffloadManager:
    def __init__(self, page_bytes: int, host_pages: int, channels: int = 8):
        lib = _native.cam()
        lib.umdk_kv_create.restype = ctypes.c_void_p
        lib.umdk_kv_host_pool.restype = ctypes.c_void_p
        lib.umdk_kv_copy_stream.restype = ctypes.c_void_p
        self._lib = lib
        self._h = ctypes.c_void_p(lib.umdk_kv_create(ctypes.c_size_t(page_bytes), ctypes.c_size_t(host_pages),
                                                     channels))
        if not self._h.value:
            raise RuntimeError("umdk_kv_create failed (pinned host allocation?)")
        self.page_bytes, self.host_pages, self.channels = page_bytes, host_pages, channels

    def host_pool_ptr(self) -> int:
        return self._lib.umdk_kv_host_pool(self._h)

    def host_pool_tensor(self, dtype=torch.bfloat16) -> torch.Tensor:
        """The pinned host pool as a CPU tensor [host_pages, page_bytes / itemsize] (no copy)."""
        n = self.host_pages * self.page_bytes
        buf = (ctypes.c_uint8 * n).from_address(self.host_pool_ptr())
        t = torch.frombuffer(buf, dtype=torch.uint8)
        return t.view(dtype).reshape(self.host_pages, -1)

    def offload(self, dev_pool: torch.Tensor, dev_pages: Sequence[int], host_slots: Sequence[int]):
        rc = self._lib.umdk_kv_offload(self._h, _native.ptr(dev_pool), _iarr(dev_pages), _iarr(host_slots),
                                       len(dev_pages), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_kv_offload failed: {rc}")

    def prefetch(self, channel: int, dev_pool: torch.Tensor, dev_pages, host_slots, n: int = None):
        """dev_pages / host_slots: sequences of ints or prebuilt ctypes int arrays (reused across steps)."""
        if not isinstance(dev_pages, ctypes.Array):
            dev_pages, host_slots = _iarr(dev_pages), _iarr(host_slots)
        n = len(dev_pages) if n is None else n
        rc = self._lib.umdk_kv_prefetch(self._h, channel, _native.ptr(dev_pool), dev_pages, host_slots, n)
        if rc != 0:
            raise RuntimeError(f"umdk_kv_prefetch failed: {rc}")

    def wait(self, channel: int):
        rc = self._lib.umdk_kv_wait(self._h, channel, _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_kv_wait failed: {rc}")

    def release(self, channel: int):
        rc = self._lib.umdk_kv_release(self._h, channel, _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_kv_release failed: {rc}")

    def sync(self):
        self._lib.umdk_kv_sync(self._h)

    def stats(self):
        out = (ctypes.c_ulonglong * 3)()
        self._lib.umdk_kv_stats(self._h, out)
        return {"bytes_h2d": int(out[0]), "bytes_d2h": int(out[1]), "copies": int(out[2])}

    def close(self):
        if self._h and self._h.value:
            self._lib.umdk_kv_destroy(self._h)
            self._h = ctypes.c_void_p()
