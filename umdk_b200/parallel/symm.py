"""Symmetric heap: one device slab per rank, mapped into every peer of the box through CUDA IPC.

B200 counterpart of the HCCL window (``windowsIn`` / ``windowsExp`` peer pointer table) that the reference's kernels
read from ``HcclOpResParam`` (src/cam/comm_operator/ascend_kernels/utils/op_kernel/moe_distribute_base.h:123-173).
Kernels receive the table of peer base pointers and use plain loads / stores / atomics on them over NVLink.

Two modes:
  * ``SymmetricHeap(nbytes, group)``: one process per GPU; handles are exchanged over the (NCCL or gloo) group.
  * ``SymmetricHeap.virtual(nbytes, num_ranks)``: all "ranks" live in this process on the current GPU. Used to run
    multi-rank protocols on a single GPU by launching the send phase of every rank before any receive phase.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _native


class SymmetricHeap:
    def __init__(self, nbytes: int, group: Optional[dist.ProcessGroup] = None):
        lib = _native.cam()
        self.nbytes = int(nbytes)
        self.group = group
        self.rank = dist.get_rank(group) if (group is not None or dist.is_initialized()) else 0
        self.world = dist.get_world_size(group) if (group is not None or dist.is_initialized()) else 1
        self._lib = lib
        self._local = ctypes.c_void_p()
        rc = lib.umdk_symm_alloc(ctypes.c_size_t(self.nbytes), ctypes.byref(self._local))
        if rc != 0:
            raise RuntimeError(f"umdk_symm_alloc({self.nbytes}) failed: {rc}")
        self._imported: List[int] = []
        self.peer_ptrs: List[int] = [0] * self.world
        self.peer_ptrs[self.rank] = self._local.value
        if self.world > 1:
            hbytes = lib.umdk_ipc_handle_bytes()
            buf = ctypes.create_string_buffer(hbytes)
            rc = lib.umdk_symm_export(self._local, buf)
            if rc != 0:
                raise RuntimeError(f"cudaIpcGetMemHandle failed: {rc}")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(buf.raw), group=group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                out = ctypes.c_void_p()
                rc = lib.umdk_symm_import(ctypes.c_char_p(h), ctypes.byref(out))
                if rc != 0:
                    raise RuntimeError(f"cudaIpcOpenMemHandle(rank {r}) failed: {rc}")
                self.peer_ptrs[r] = out.value
                self._imported.append(out.value)
            dist.barrier(group=group)
        self._virtual_children: List["SymmetricHeap"] = []

    @classmethod
    def virtual(cls, nbytes: int, num_ranks: int) -> List["SymmetricHeap"]:
        """R heaps on the current device that all see each other (single process)."""
        lib = _native.cam()
        heaps = []
        ptrs = []
        for _ in range(num_ranks):
            p = ctypes.c_void_p()
            rc = lib.umdk_symm_alloc(ctypes.c_size_t(int(nbytes)), ctypes.byref(p))
            if rc != 0:
                raise RuntimeError(f"umdk_symm_alloc failed: {rc}")
            ptrs.append(p.value)
        for r in range(num_ranks):
            h = cls.__new__(cls)
            h.nbytes = int(nbytes)
            h.group = None
            h.rank = r
            h.world = num_ranks
            h._lib = lib
            h._local = ctypes.c_void_p(ptrs[r])
            h._imported = []
            h.peer_ptrs = list(ptrs)
            h._virtual_children = []
            h.is_virtual = True
            heaps.append(h)
        return heaps

    @classmethod
    def multicast(cls, nbytes: int, group: Optional[dist.ProcessGroup] = None) -> "SymmetricHeap":
        """Heap whose slabs are also bound to an NVLink multicast object (NVLS): besides the per-peer pointers it
        offers ``multicast_ptr``, an address on which ``multimem`` loads reduce over all ranks inside NVSwitch and
        ``multimem`` stores broadcast to all ranks. Allocation and handle exchange go through
        ``torch.distributed._symmetric_memory`` (plumbing only; the kernels that use the pointers are this
        package's). Raises if the platform cannot provide a multicast mapping."""
        import torch.distributed._symmetric_memory as symm_mem
        pg = group if group is not None else dist.group.WORLD
        dev = torch.device("cuda", torch.cuda.current_device())
        t = symm_mem.empty(int(nbytes), dtype=torch.uint8, device=dev)
        hdl = symm_mem.rendezvous(t, pg)
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        if mc == 0:
            raise RuntimeError("no NVLink multicast mapping available for this group")
        t.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=group)
        h = cls.__new__(cls)
        h.nbytes = int(nbytes)
        h.group = group
        h.rank = dist.get_rank(group)
        h.world = dist.get_world_size(group)
        h._lib = _native.cam()
        h._local = ctypes.c_void_p(int(hdl.buffer_ptrs[h.rank]))
        h._imported = []
        h.peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
        h.multicast_ptr = mc
        h._torch_keepalive = (t, hdl)
        h._virtual_children = []
        return h

    @property
    def local_ptr(self) -> int:
        return self._local.value

    def peer_array(self, n: int = 32):
        arr = (ctypes.c_void_p * n)()
        for i, p in enumerate(self.peer_ptrs):
            arr[i] = p
        return arr

    def close(self):
        lib = self._lib
        if getattr(self, "_torch_keepalive", None) is not None:
            self._torch_keepalive = None  # memory is owned by torch's symmetric-memory allocator
            self._local = ctypes.c_void_p()
            return
        for p in self._imported:
            lib.umdk_symm_unimport(ctypes.c_void_p(p))
        self._imported = []
        if self._local and self._local.value:
            lib.umdk_symm_free(self._local)
            self._local = ctypes.c_void_p()


class HostMirror:
    """Small pinned host buffer that kernels can store to (receive counts), polled by the CPU."""

    def __init__(self, nints: int = 8):
        lib = _native.cam()
        self._lib = lib
        self._h = ctypes.c_void_p()
        self._d = ctypes.c_void_p()
        rc = lib.umdk_host_mapped_alloc(ctypes.c_size_t(nints * 4), ctypes.byref(self._h), ctypes.byref(self._d))
        if rc != 0:
            raise RuntimeError(f"umdk_host_mapped_alloc failed: {rc}")
        self.host = (ctypes.c_int * nints).from_address(self._h.value)
        self.dev_ptr = self._d.value

    def close(self):
        if self._h and self._h.value:
            self._lib.umdk_host_mapped_free(self._h)
            self._h = ctypes.c_void_p()
