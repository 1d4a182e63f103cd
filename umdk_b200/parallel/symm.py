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
        ``multimem`` stores broadcast to all ranks. Built on the driver's virtual-memory-management calls
        (csrc/cam/symm_mc.cu): every rank creates its memory, the descriptors travel between the processes with
        pidfd_getfd, rank 0 creates the multicast object, all ranks join, bind and map it. Raises when the GPUs or
        the driver cannot do multicast; callers then stay on the peer-pointer algorithms."""
        lib = _native.cam()
        pg = group if group is not None else dist.group.WORLD
        rank, world = dist.get_rank(pg), dist.get_world_size(pg)
        # every rank must take the same branch: agree first
        ok = torch.tensor([int(lib.umdk_mc_supported())], dtype=torch.int32, device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=pg)
        if int(ok.item()) == 0:
            raise RuntimeError("no NVLink multicast support on this group's GPUs")
        import os
        heap, local = ctypes.c_void_p(), ctypes.c_void_p()
        fd, padded = ctypes.c_int(-1), ctypes.c_size_t(0)

        def agree(rc: int, what: str):
            """Raises on EVERY rank when the step failed on any rank (a rank that went on alone would wait forever)."""
            t = torch.tensor([int(rc != 0)], dtype=torch.int32, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=pg)
            if int(t.item()):
                if heap.value:
                    lib.umdk_mc_destroy(heap)
                raise RuntimeError(f"multicast heap: {what} failed (rc {rc} on rank {rank})")

        agree(lib.umdk_mc_local_create(ctypes.c_size_t(int(nbytes)), world, ctypes.byref(heap), ctypes.byref(local),
                                       ctypes.byref(fd), ctypes.byref(padded)), "local allocation")
        mc_fd = ctypes.c_int(-1)
        rc = lib.umdk_mc_group_create(heap, ctypes.byref(mc_fd)) if rank == 0 else 0
        agree(rc, "multicast object creation")
        # (pid, descriptor of the local memory, descriptor of the multicast object on rank 0) of every rank
        infos = [None] * world
        dist.all_gather_object(infos, (os.getpid(), fd.value, mc_fd.value), group=pg)
        rc = 0
        if rank != 0:
            got = lib.umdk_fd_from_process(infos[0][0], infos[0][2])
            rc = lib.umdk_mc_group_import(heap, got) if got >= 0 else got
            if got >= 0:
                os.close(got)
        agree(rc, "multicast object import")
        agree(lib.umdk_mc_add_device(heap), "joining the multicast object")      # all joined before anyone binds
        mc_ptr = ctypes.c_void_p()
        agree(lib.umdk_mc_bind_map(heap, ctypes.byref(mc_ptr)), "binding / mapping the multicast object")
        peer_ptrs, rc = [0] * world, 0
        for r in range(world):
            if r == rank:
                peer_ptrs[r] = local.value
                continue
            got = lib.umdk_fd_from_process(infos[r][0], infos[r][1])
            p = ctypes.c_void_p()
            rc = rc or (lib.umdk_mc_import_peer(heap, got, ctypes.byref(p)) if got >= 0 else got)
            if got >= 0:
                os.close(got)
            peer_ptrs[r] = p.value or 0
        agree(rc, "mapping the peers' memory")     # also: nobody closes its descriptors before all have duplicated them
        h = cls.__new__(cls)
        h.nbytes = int(nbytes)
        h.group = group
        h.rank, h.world = rank, world
        h._lib = lib
        h._local = ctypes.c_void_p(local.value)
        h._imported = []
        h.peer_ptrs = peer_ptrs
        h.multicast_ptr = mc_ptr.value
        h._mc_heap = heap
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
        if getattr(self, "_mc_heap", None) is not None:   # unmaps the peers, the multicast range and the local memory
            lib.umdk_mc_destroy(self._mc_heap)
            self._mc_heap = None
            self._local = ctypes.c_void_p()
            self.multicast_ptr = 0
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
