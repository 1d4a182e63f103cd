"""KV-cache offload / prefetch manager (csrc/cam/kv_offload.cu): pinned host pool, cudaMemcpyAsync of whole pages on a
side stream, and a row-granular gather prefetch (only the token rows that sparse attention selected) on the same
stream."""
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
        lib.umdk_kv_create_on_stream.restype = ctypes.c_void_p
        lib.umdk_kv_host_pool.restype = ctypes.c_void_p
        lib.umdk_kv_copy_stream.restype = ctypes.c_void_p
        self._lib = lib
        # the side stream belongs to torch's stream pool, so tensors staged on it never outlive it
        self._stream = torch.cuda.Stream()
        self._h = ctypes.c_void_p(lib.umdk_kv_create_on_stream(ctypes.c_size_t(page_bytes),
                                                               ctypes.c_size_t(host_pages), channels,
                                                               ctypes.c_void_p(self._stream.cuda_stream)))
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

    def prefetch_rows(self, channel: int, indices: torch.Tensor, host_table: torch.Tensor, landing: torch.Tensor,
                      indices_out: torch.Tensor, virt_base: int, page_tokens: int, status: torch.Tensor = None,
                      after_compute: bool = True, num_ctas: int = 8):
        """Fetches the selected rows that live in host pages into ``landing`` ([B * topk, row] device rows) and writes
        ``indices_out``: the position itself for rows of device pages, ``virt_base + i`` for landed rows.
        indices [B, topk] int32 (device), host_table [B, n_logical_pages] int32 (device; host slot or -1).
        ``after_compute``: order the gather after everything queued on the current stream (which produced the
        indices); False when the indices are already final or were written on ``side_stream()``."""
        assert indices.is_cuda and indices.dtype == torch.int32 and indices.is_contiguous()
        assert host_table.is_cuda and host_table.dtype == torch.int32 and host_table.is_contiguous()
        assert indices_out.shape == indices.shape and indices_out.dtype == torch.int32 and indices_out.is_contiguous()
        B, topk = indices.shape
        row_bytes = self.page_bytes // page_tokens
        assert landing.is_contiguous() and landing.numel() * landing.element_size() >= B * topk * row_bytes
        self._lib.umdk_kv_rows_fetched.restype = ctypes.c_longlong
        rc = self._lib.umdk_kv_prefetch_rows(self._h, channel, _native.ptr(indices), _native.ptr(host_table),
                                             _native.ptr(landing), _native.ptr(indices_out), B, topk,
                                             host_table.shape[1], page_tokens, row_bytes, virt_base,
                                             _native.ptr(status), 1 if after_compute else 0, num_ctas,
                                             _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_kv_prefetch_rows failed: {rc}")

    def side_stream(self) -> torch.cuda.Stream:
        """The manager's copy stream as a torch stream (to stage inputs of a prefetch on it)."""
        return self._stream

    def rows_fetched(self) -> int:
        """Host rows moved by prefetch_rows since creation (waits for the side stream)."""
        self._lib.umdk_kv_rows_fetched.restype = ctypes.c_longlong
        return int(self._lib.umdk_kv_rows_fetched(self._h))

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
