"""Tensor-parallel fused ops over NVLink peer memory (csrc/cam/tp_gemm.cu, csrc/cam/allreduce.cu):
all-gather -> GEMM, GEMM -> reduce-scatter, and one-/two-shot all-reduce."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native
from ..parallel.symm import SymmetricHeap
from .ep import Recoverable, check_status
from ..utils import trace as _trace

MAX_RANKS = 32


class _TpParams(ctypes.Structure):
    _fields_ = [
        ("mode", ctypes.c_int), ("R", ctypes.c_int), ("rank", ctypes.c_int), ("Ts", ctypes.c_int),
        ("N", ctypes.c_int), ("K", ctypes.c_int), ("n_copy", ctypes.c_int), ("max_ctas", ctypes.c_int),
        ("peers", ctypes.c_void_p * MAX_RANKS),
        ("x_slot_off", ctypes.c_uint64 * 2), ("ready_off", ctypes.c_uint64 * 2), ("recv_off", ctypes.c_uint64 * 2),
        ("arrive_off", ctypes.c_uint64),
        ("a_local", ctypes.c_void_p), ("xg", ctypes.c_void_p), ("w", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("chunk_done", ctypes.c_void_p), ("ctrl", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("phase_mask", ctypes.c_int), ("impl", ctypes.c_int),
    ]


class _ArParams(ctypes.Structure):
    _fields_ = [
        ("R", ctypes.c_int), ("rank", ctypes.c_int), ("algo", ctypes.c_int), ("num_ctas", ctypes.c_int),
        ("phase_mask", ctypes.c_int),
        ("peers", ctypes.c_void_p * MAX_RANKS),
        ("buf_off", ctypes.c_uint64 * 2), ("flag_off", ctypes.c_uint64),
        ("inp", ctypes.c_void_p), ("out", ctypes.c_void_p), ("n", ctypes.c_ulonglong),
        ("ctrl", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("mc_base", ctypes.c_void_p), ("in_place", ctypes.c_int), ("buf_bytes", ctypes.c_ulonglong),
    ]


def _align(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class TpComm(Recoverable):
    """Per-rank state of the fused tensor-parallel GEMMs for fixed shard sizes.

    ``ag_gemm(x_shard [Ts, K], w [N, K]) -> [R*Ts, N]`` and ``gemm_rs(y [R*Ts, Kr], w [N, Kr]) -> [Ts, N]``.
    """

    _epoch_words = {"ctrl_ag": (0,), "ctrl_rs": (0,)}
    _zero_between_calls = ("chunk_done",)

    def __init__(self, heap: SymmetricHeap, ts: int, k_ag: int, n_rs: int, n_copy: int = 0, max_ctas: int = 0,
                 single_cta: bool = False):
        self.lib = _native.cam()
        self.heap, self.R, self.rank = heap, heap.world, heap.rank
        self.Ts, self.K_ag, self.N_rs = ts, k_ag, n_rs
        need = self.heap_bytes(self.R, ts, k_ag, n_rs)
        if need > heap.nbytes:
            raise ValueError(f"symmetric heap too small: need {need}, have {heap.nbytes}")
        off = 0
        shard = _align(ts * k_ag * 2, 1024)
        self.x_slot = (off, off + shard)
        off += 2 * shard
        fl = _align(self.R * 8, 256)
        self.ready = (off, off + fl)
        off += 2 * fl
        rv = _align(self.R * ts * n_rs * 2, 1024)
        self.recv = (off, off + rv)
        off += 2 * rv
        self.arrive = off
        dev = torch.device("cuda", torch.cuda.current_device())
        self.ctrl_ag = torch.zeros(8, dtype=torch.int32, device=dev)
        self.ctrl_rs = torch.zeros(8, dtype=torch.int32, device=dev)
        self.chunk_done = torch.zeros(self.R, dtype=torch.int32, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self.xg = torch.empty(self.R * ts, k_ag, dtype=torch.bfloat16, device=dev)
        # CTAs that only move peer shards (all-gather -> GEMM). Each one is taken from the GEMM, but fewer than 16 made
        # the GEMM wait for its remote chunks even on 2 GPUs (4 copy CTAs: 3363 us against 2915 us with 16).
        if n_copy <= 0:
            n_copy = 16
        self.n_copy, self.max_ctas = n_copy, max_ctas
        # False: CTA pairs (256 x 256 tiles) where Ts and N are multiples of 256; True: always one CTA per tile
        self.single_cta = single_cta

    @staticmethod
    def heap_bytes(R: int, ts: int, k_ag: int, n_rs: int) -> int:
        lib = _native.cam()
        lib.umdk_tp_heap_bytes.restype = ctypes.c_longlong
        n = lib.umdk_tp_heap_bytes(R, ts, k_ag, n_rs)
        if n < 0:
            raise ValueError("unsupported tensor-parallel geometry")
        return int(n)

    def _params(self, mode: int) -> _TpParams:
        p = _TpParams()
        p.mode, p.R, p.rank, p.Ts = mode, self.R, self.rank, self.Ts
        p.n_copy, p.max_ctas = self.n_copy, self.max_ctas
        p.impl = 1 if self.single_cta else 0
        for i, pp in enumerate(self.heap.peer_ptrs):
            p.peers[i] = pp
        p.x_slot_off[0], p.x_slot_off[1] = self.x_slot
        p.ready_off[0], p.ready_off[1] = self.ready
        p.recv_off[0], p.recv_off[1] = self.recv
        p.arrive_off = self.arrive
        p.status = self.status.data_ptr()
        return p

    @_trace.traced("umdk.tp.ag_gemm")
    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                phase_mask: int = 3) -> torch.Tensor:
        self._guard()
        assert x_shard.dtype == torch.bfloat16 and x_shard.is_contiguous() and w.is_contiguous()
        assert x_shard.shape == (self.Ts, self.K_ag) and w.shape[1] == self.K_ag
        N = w.shape[0]
        if out is None:
            out = torch.empty(self.R * self.Ts, N, dtype=torch.bfloat16, device=x_shard.device)
        p = self._params(0)
        p.N, p.K = N, self.K_ag
        p.a_local, p.xg, p.w, p.out = x_shard.data_ptr(), self.xg.data_ptr(), w.data_ptr(), out.data_ptr()
        p.chunk_done, p.ctrl = self.chunk_done.data_ptr(), self.ctrl_ag.data_ptr()
        p.phase_mask = phase_mask
        rc = self.lib.umdk_tp_gemm(ctypes.byref(p), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_tp_gemm(all-gather GEMM) failed: {rc}")
        return out

    @_trace.traced("umdk.tp.gemm_rs")
    def gemm_rs(self, y: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                phase_mask: int = 3) -> torch.Tensor:
        self._guard()
        assert y.dtype == torch.bfloat16 and y.is_contiguous() and w.is_contiguous()
        assert y.shape[0] == self.R * self.Ts and w.shape == (self.N_rs, y.shape[1])
        if out is None:
            out = torch.empty(self.Ts, self.N_rs, dtype=torch.bfloat16, device=y.device)
        p = self._params(1)
        p.N, p.K = self.N_rs, y.shape[1]
        p.a_local, p.w, p.out = y.data_ptr(), w.data_ptr(), out.data_ptr()
        p.ctrl = self.ctrl_rs.data_ptr()
        p.phase_mask = phase_mask
        rc = self.lib.umdk_tp_gemm(ctypes.byref(p), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_tp_gemm(GEMM reduce-scatter) failed: {rc}")
        return out

    def check(self):
        check_status(self.status, "tp_gemm", owner=self)


class AllReduce(Recoverable):
    """bf16 sum all-reduce over NVLink peer memory. ``algo``: 'one_shot' (every rank loads all peers' data),
    'two_shot' (reduce-scatter + all-gather with peer loads), 'push' (the same two stages with peer STORES only; needs
    buffers of twice the message size), 'nvls' (multimem reduce / broadcast inside NVSwitch; multicast heap), or
    'one_shot_push' (every rank stores its vector into a slot on every peer, then sums locally; needs world x the
    message size), or 'auto' (by size and heap kind)."""

    _epoch_words = {"ctrl": (0,)}

    def reset(self, epoch=None, group=None) -> int:
        epoch = super().reset(epoch, group)
        self.calls = epoch   # the host mirror of the device epoch picks the buffer parity of the next call
        return epoch

    def __init__(self, heap: SymmetricHeap, max_bytes: int):
        self.lib = _native.cam()
        self.heap, self.R, self.rank = heap, heap.world, heap.rank
        self.max_bytes = max_bytes
        if self.heap_bytes(max_bytes, self.R) > heap.nbytes:
            raise ValueError("symmetric heap too small for the all-reduce buffers")
        b = _align(max_bytes, 1024)
        self.buf = (0, b)
        self.flag = 2 * b
        dev = torch.device("cuda", torch.cuda.current_device())
        self.ctrl = torch.zeros(8, dtype=torch.int32, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self.calls = 0  # host mirror of the device epoch (buffer parity of the next call = calls & 1)

    @property
    def next_parity(self) -> int:
        return self.calls & 1

    @staticmethod
    def heap_bytes(max_bytes: int, R: int) -> int:
        lib = _native.cam()
        lib.umdk_allreduce_heap_bytes.restype = ctypes.c_longlong
        return int(lib.umdk_allreduce_heap_bytes(ctypes.c_ulonglong(max_bytes), R))

    def buffer(self, n: int, parity: int) -> torch.Tensor:
        """bf16 view of the heap buffer of the given epoch parity: fill it and call with ``in_place=True`` to skip
        the copy-in / copy-out (the result replaces the input in that buffer)."""
        from ..utils.rawtensor import from_ptr
        return from_ptr(self.heap.local_ptr + self.buf[parity], (n,), torch.bfloat16, self.ctrl.device)

    @_trace.traced("umdk.tp.all_reduce")
    def __call__(self, x: Optional[torch.Tensor], out: Optional[torch.Tensor] = None, algo: str = "auto",
                 num_ctas: int = 0, phase_mask: int = 3, in_place: bool = False, n: Optional[int] = None
                 ) -> Optional[torch.Tensor]:
        self._guard()
        if not in_place:
            assert x.dtype == torch.bfloat16 and x.is_contiguous()
            n = x.numel()
            if out is None:
                out = torch.empty_like(x)
        assert n * 2 <= self.max_bytes and n % (8 * self.R) == 0, "size must be a multiple of 8 * world elements"
        has_mc = getattr(self.heap, "multicast_ptr", 0) != 0
        if algo == "auto":
            # measured on 2 and 8 GPUs: store-only variants win wherever their staging fits; in-switch reduction wins
            # for large messages on more than two GPUs
            if n * 2 <= (4 << 20):
                algo = "one_shot_push" if 2 * n * self.R <= self.max_bytes else "one_shot"
            elif has_mc and self.R > 2:
                algo = "nvls"
            else:
                algo = "push" if 4 * n <= self.max_bytes else "two_shot"
        code = {"one_shot": 0, "two_shot": 1, "nvls": 2, "push": 3, "one_shot_push": 4}[algo]
        if code == 4:
            assert 2 * n * self.R <= self.max_bytes, "'one_shot_push' needs max_bytes >= world x the message size"
        if code == 3:
            assert 4 * n <= self.max_bytes, "'push' needs max_bytes >= 2 x the message size"
            if phase_mask == 3:
                phase_mask = 7
        p = _ArParams()
        p.R, p.rank, p.algo, p.num_ctas, p.phase_mask = self.R, self.rank, code, num_ctas, phase_mask
        p.mc_base = getattr(self.heap, "multicast_ptr", 0) or None
        p.in_place = int(in_place)
        for i, pp in enumerate(self.heap.peer_ptrs):
            p.peers[i] = pp
        p.buf_off[0], p.buf_off[1] = self.buf
        p.flag_off = self.flag
        p.inp = x.data_ptr() if x is not None else None
        p.out = out.data_ptr() if out is not None else None
        p.n = n
        p.ctrl, p.status = self.ctrl.data_ptr(), self.status.data_ptr()
        p.buf_bytes = _align(self.max_bytes, 1024)
        rc = self.lib.umdk_allreduce(ctypes.byref(p), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_allreduce failed: {rc}")
        if phase_mask & (4 if code == 3 else 2):
            self.calls += 1
        return out

    def check(self):
        check_status(self.status, "allreduce", owner=self)
