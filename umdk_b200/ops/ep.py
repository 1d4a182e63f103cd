"""Normal-mode expert-parallel dispatch / combine on the GPU (hand-written sm_100a kernels in csrc/cam/ep_normal.cu).

``EpNormal`` owns the per-geometry state one rank needs: its slice of the symmetric heap, the control words
(epochs, arrival counters), the layout scratch and the status record that kernels fill when a bounded wait runs
out. The public, user-facing surface is :class:`umdk_b200.buffer.Buffer` and the ``umdk_cam_op_lib`` torch ops; this
module is the thin layer between them and the C entry points.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import _native
from ..parallel.symm import HostMirror, SymmetricHeap
from ..utils import trace as _trace

MAX_RANKS = 32


class _DispatchParams(ctypes.Structure):
    _fields_ = [
        ("R", ctypes.c_int), ("rank", ctypes.c_int), ("E", ctypes.c_int), ("K", ctypes.c_int), ("H", ctypes.c_int),
        ("cap", ctypes.c_int), ("quant", ctypes.c_int), ("T", ctypes.c_int),
        ("n_cap", ctypes.c_int), ("a_cap", ctypes.c_int), ("num_ctas", ctypes.c_int), ("phase_mask", ctypes.c_int),
        ("peers", ctypes.c_void_p * MAX_RANKS),
        ("x", ctypes.c_void_p), ("topk_idx", ctypes.c_void_p), ("topk_w", ctypes.c_void_p),
        ("send_idx", ctypes.c_void_p), ("rank_slot", ctypes.c_void_p), ("num_per_expert", ctypes.c_void_p),
        ("num_per_rank", ctypes.c_void_p),
        ("recv_x", ctypes.c_void_p), ("recv_scales", ctypes.c_void_p), ("expand_idx", ctypes.c_void_p),
        ("recv_count", ctypes.c_void_p), ("recv_per_expert", ctypes.c_void_p), ("recv_meta", ctypes.c_void_p),
        ("counts_dev", ctypes.c_void_p), ("counts_host", ctypes.c_void_p),
        ("ctrl", ctypes.c_void_p), ("status", ctypes.c_void_p), ("diag", ctypes.c_void_p),
    ]


class _CombineParams(ctypes.Structure):
    _fields_ = [
        ("R", ctypes.c_int), ("rank", ctypes.c_int), ("E", ctypes.c_int), ("K", ctypes.c_int), ("H", ctypes.c_int),
        ("cap", ctypes.c_int), ("T", ctypes.c_int),
        ("mode", ctypes.c_int), ("apply_weights", ctypes.c_int), ("n_rows", ctypes.c_int),
        ("num_ctas", ctypes.c_int), ("phase_mask", ctypes.c_int),
        ("peers", ctypes.c_void_p * MAX_RANKS),
        ("y", ctypes.c_void_p), ("recv_meta", ctypes.c_void_p), ("counts_dev", ctypes.c_void_p),
        ("src_idx", ctypes.c_void_p), ("in_rank", ctypes.c_void_p), ("topk_idx", ctypes.c_void_p),
        ("topk_w", ctypes.c_void_p), ("out", ctypes.c_void_p), ("ctrl", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("diag", ctypes.c_void_p),
    ]


class _NotifyParams(ctypes.Structure):
    _fields_ = [
        ("R", ctypes.c_int), ("rank", ctypes.c_int), ("E", ctypes.c_int), ("K", ctypes.c_int), ("H", ctypes.c_int),
        ("cap", ctypes.c_int), ("phase_mask", ctypes.c_int),
        ("peers", ctypes.c_void_p * MAX_RANKS),
        ("num_per_expert", ctypes.c_void_p), ("num_per_rank", ctypes.c_void_p),
        ("recv_count", ctypes.c_void_p), ("recv_offset", ctypes.c_void_p), ("recv_per_expert", ctypes.c_void_p),
        ("totals", ctypes.c_void_p), ("ctrl", ctypes.c_void_p), ("status", ctypes.c_void_p),
    ]


class KernelStatusError(RuntimeError):
    """A kernel gave up on a bounded wait or rejected an out-of-range index; the record says where."""


_PHASES = {1: "tma-empty", 2: "tma-full", 3: "tmem-full", 4: "tmem-empty", 5: "dispatch-count", 6: "dispatch-data",
           7: "combine-data", 8: "grid-barrier", 9: "group-ready", 10: "allreduce", 11: "ag-chunk", 12: "rs-chunk"}
_CODES = {1: "timeout", 2: "bad-argument", 3: "overflow", 4: "cuda-error"}


def check_status(status: torch.Tensor, what: str = "kernel", owner=None):
    """Reads the 4-int status record (synchronises) and raises if a kernel reported an error. ``owner`` (an object
    with the ``Recoverable`` mix-in) is marked poisoned: a kernel that gave up on a wait may have left its shared
    counters and epoch words half-updated, so further launches are refused until ``owner.reset()``."""
    s = status.tolist()
    if s[0] != 0:
        status.zero_()
        msg = (f"{what}: {_CODES.get(s[0], s[0])} in phase {_PHASES.get(s[1], s[1])} "
               f"(detail {s[2]}, {s[3]})")
        if owner is not None:
            owner._poisoned = msg
        raise KernelStatusError(msg)


class Recoverable:
    """Mix-in for objects that own device-side protocol state (control words with epoch counters, arrival counters,
    grid-barrier words). After a kernel reported a time-out, arrival counters may hold a partial count and the ranks'
    epochs may differ; carrying on would make the next call's "last CTA" fire early or a flag wait pass on stale data.
    So ``check()`` poisons the object, every launch method calls ``_guard()`` first, and ``reset()`` puts the state
    back: all counters zero, every epoch word set to a value above anything any rank has used (agreed over the
    process group, or passed in by a caller that drives several virtual ranks in one process)."""

    _poisoned: Optional[str] = None
    # attribute name of an int32 control tensor -> indices of its epoch words; other words are counters
    _epoch_words: dict = {}
    # further int32 / int64 tensors that must be zero between calls
    _zero_between_calls: tuple = ()

    def _guard(self):
        if self._poisoned is not None:
            raise KernelStatusError(f"object is poisoned by an earlier kernel error ({self._poisoned}); call reset()")

    def max_epoch(self) -> int:
        m = 0
        for name, words in self._epoch_words.items():
            t = getattr(self, name)
            for i in words:
                m = max(m, int(t[i].item()) & 0x7fffffff)
        return m

    def reset(self, epoch: Optional[int] = None, group=None) -> int:
        """Clears the poison. Every rank of the group must call it (it synchronises the device and, with a process
        group, the ranks). Returns the epoch now in force."""
        import torch.distributed as dist
        torch.cuda.synchronize()
        if epoch is None:
            epoch = self.max_epoch() + 2
            heap = getattr(self, "heap", None)
            group = group if group is not None else getattr(heap, "group", None)
            if dist.is_initialized() and heap is not None and heap.world > 1 and not getattr(heap, "is_virtual", False):
                t = torch.tensor([epoch], dtype=torch.int64, device=self.status.device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
                epoch = int(t.item())
        for name, words in self._epoch_words.items():
            t = getattr(self, name)
            t.zero_()
            for i in words:
                t[i] = epoch
        for name in self._zero_between_calls:
            getattr(self, name).zero_()
        self.status.zero_()
        torch.cuda.synchronize()
        heap = getattr(self, "heap", None)
        if dist.is_initialized() and heap is not None and heap.world > 1 and not getattr(heap, "is_virtual", False):
            dist.barrier(group=group)
        self._poisoned = None
        return epoch


@dataclass
class LayoutResult:
    num_tokens_per_expert: torch.Tensor
    num_tokens_per_rank: torch.Tensor
    is_token_in_rank: torch.Tensor
    send_token_idx: torch.Tensor
    rank_slot: torch.Tensor


@dataclass
class NotifyResult:
    """What a rank learns from the count exchange before any token moves (the outputs of the reference's
    notify_dispatch operator: notify_dispatch.h:91-160)."""
    recv_count: torch.Tensor              # [E_local * R] inclusive prefix over (local expert, source rank)
    recv_offset: torch.Tensor             # [E_local * R] exclusive prefix
    recv_tokens_per_expert: torch.Tensor  # [E_local] int64
    totals: torch.Tensor                  # [4] int32: rows to receive, tokens to receive, max tokens from one source


@dataclass
class DispatchResult:
    recv_x: torch.Tensor                 # [n_cap, H] fp8 (uint8 storage viewed as float8_e4m3fn) or bf16
    recv_scales: Optional[torch.Tensor]  # [n_cap, H/128] fp32
    expand_idx: torch.Tensor             # [n_cap, 3]
    recv_count: torch.Tensor             # [E_local * R] inclusive prefix
    recv_tokens_per_expert: torch.Tensor # [E_local] int64
    recv_meta: torch.Tensor              # [a_cap, 2K+2]
    counts: torch.Tensor                 # device [4 + 32]: rows N, arrivals A, max from one source, 0; then the
                                         # index of the first arrival of every source rank
    layout: LayoutResult
    topk_idx: torch.Tensor
    topk_weights: Optional[torch.Tensor]
    num_tokens: int
    quant: bool
    num_recv: Optional[int] = None       # host value of N when the caller asked for it


def layout(topk_idx: torch.Tensor, num_experts: int, num_ranks: int, scratch=None, bar=None, status=None,
           out: Optional[LayoutResult] = None) -> LayoutResult:
    """GPU ``get_dispatch_layout``: stable bucket positions per expert and per destination rank. ``out`` reuses the
    tensors of an earlier result of the same shape (no allocations on the call path)."""
    lib = _native.cam()
    assert topk_idx.is_cuda and topk_idx.dtype == torch.int64 and topk_idx.is_contiguous()
    T, K = topk_idx.shape
    dev = topk_idx.device
    E, R = num_experts, num_ranks
    if out is not None:
        npe, npr, sidx, rslot = out.num_tokens_per_expert, out.num_tokens_per_rank, out.send_token_idx, out.rank_slot
        inr = out.is_token_in_rank.view(torch.uint8)
        assert sidx.shape == (T, K) and rslot.shape == (T, R) and npe.numel() == E
    else:
        npe = torch.empty(E, dtype=torch.int32, device=dev)
        npr = torch.empty(R, dtype=torch.int32, device=dev)
        inr = torch.empty(T, R, dtype=torch.uint8, device=dev)
        sidx = torch.empty(T, K, dtype=torch.int32, device=dev)
        rslot = torch.empty(T, R, dtype=torch.int32, device=dev)
    chunks = (T + 31) // 32
    if scratch is None or scratch.numel() < max(1, chunks) * (E + R):
        scratch = torch.empty(max(1, chunks) * (E + R), dtype=torch.int32, device=dev)
    if bar is None:
        bar = torch.zeros(2, dtype=torch.int32, device=dev)
    if status is None:
        status = torch.zeros(4, dtype=torch.int32, device=dev)
    rc = lib.umdk_ep_layout(_native.ptr(topk_idx), T, K, E, R, _native.ptr(npe), _native.ptr(npr), _native.ptr(inr),
                            _native.ptr(sidx), _native.ptr(rslot), _native.ptr(scratch), _native.ptr(bar),
                            _native.ptr(status), _native.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"umdk_ep_layout failed: {rc}")
    return out if out is not None else LayoutResult(npe, npr, inr.view(torch.bool), sidx, rslot)


class EpNormal(Recoverable):
    """State of one rank for normal-mode dispatch / combine at a fixed geometry (E, K, H, cap)."""

    _epoch_words = {"ctrl": (0, 3, 8)}      # dispatch, combine, notify epochs (ep_normal.cu)
    _zero_between_calls = ("layout_bar",)

    def __init__(self, heap: SymmetricHeap, num_experts: int, top_k: int, hidden: int, cap: int,
                 num_ctas: int = 0, device=None):
        self.lib = _native.cam()
        self.heap = heap
        self.R, self.rank = heap.world, heap.rank
        self.E, self.K, self.H, self.cap = num_experts, top_k, hidden, cap
        self.num_ctas = num_ctas
        need = self.heap_bytes(self.R, num_experts, top_k, hidden, cap)
        if need > heap.nbytes:
            raise ValueError(f"symmetric heap too small: need {need} bytes, have {heap.nbytes}")
        dev = device or torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        self.ctrl = torch.zeros(64, dtype=torch.int32, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self.layout_bar = torch.zeros(2, dtype=torch.int32, device=dev)
        self.layout_scratch = torch.empty(((cap + 31) // 32) * (num_experts + self.R), dtype=torch.int32, device=dev)
        self.mirror = HostMirror(8)
        # diagnose mode: the kernels record how long (ns) this rank waited for each source rank's data; gather the
        # rows of all ranks into a matrix and pass it to examples/utils.py:diagnose_matrix to find a slow rank or link
        # (the reference's in-kernel wait statistics: moe_dispatch_normal.h:489-529, moe_combine_normal.h:259-280)
        self.diagnose = False
        self.diag_dispatch = torch.zeros(self.R, dtype=torch.int64, device=dev)
        self.diag_combine = torch.zeros(self.R, dtype=torch.int64, device=dev)

    def wait_times_us(self):
        """(dispatch, combine) wait time per source rank in microseconds from the last diagnosed calls."""
        return self.diag_dispatch.double().cpu() / 1e3, self.diag_combine.double().cpu() / 1e3

    @staticmethod
    def heap_bytes(R: int, E: int, K: int, H: int, cap: int) -> int:
        lib = _native.cam()
        lib.umdk_ep_normal_heap_bytes.restype = ctypes.c_longlong
        n = lib.umdk_ep_normal_heap_bytes(R, E, K, H, cap)
        if n < 0:
            raise ValueError(f"unsupported EP geometry R={R} E={E} K={K} H={H} cap={cap}")
        return int(n)

    @_trace.traced("umdk.ep.layout")
    def layout(self, topk_idx: torch.Tensor, out: Optional[LayoutResult] = None) -> LayoutResult:
        return layout(topk_idx, self.E, self.R, self.layout_scratch, self.layout_bar, self.status, out=out)

    @_trace.traced("umdk.ep.notify")
    def notify(self, lay: LayoutResult, phase_mask: int = 3, out: Optional[NotifyResult] = None) -> NotifyResult:
        """Count exchange alone: tells every peer how many rows / tokens this rank will send to each of its local
        experts and returns what this rank will receive. ``dispatch`` does the same exchange internally; call this
        when the sizes are needed first (to size buffers, or to balance load) - one launch of one CTA."""
        self._guard()
        El = self.E // self.R
        if out is None:
            dev = self.device
            out = NotifyResult(torch.empty(El * self.R, dtype=torch.int32, device=dev),
                               torch.empty(El * self.R, dtype=torch.int32, device=dev),
                               torch.empty(El, dtype=torch.int64, device=dev),
                               torch.zeros(4, dtype=torch.int32, device=dev))
        p = _NotifyParams()
        p.R, p.rank, p.E, p.K, p.H, p.cap, p.phase_mask = self.R, self.rank, self.E, self.K, self.H, self.cap, phase_mask
        for i, pp in enumerate(self.heap.peer_ptrs):
            p.peers[i] = pp
        p.num_per_expert, p.num_per_rank = lay.num_tokens_per_expert.data_ptr(), lay.num_tokens_per_rank.data_ptr()
        p.recv_count, p.recv_offset = out.recv_count.data_ptr(), out.recv_offset.data_ptr()
        p.recv_per_expert, p.totals = out.recv_tokens_per_expert.data_ptr(), out.totals.data_ptr()
        p.ctrl, p.status = self.ctrl.data_ptr(), self.status.data_ptr()
        rc = self.lib.umdk_ep_notify(ctypes.byref(p), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_ep_notify failed: {rc}")
        return out

    @_trace.traced("umdk.ep.dispatch")
    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: Optional[torch.Tensor],
                 lay: Optional[LayoutResult] = None, quant: bool = True, n_cap: Optional[int] = None,
                 a_cap: Optional[int] = None, phase_mask: int = 3, out: Optional[DispatchResult] = None,
                 sync_counts: bool = False) -> DispatchResult:
        """Runs notify + quantise + push + expand. ``phase_mask`` 1 / 2 run only the send / receive half (used to
        drive several virtual ranks from one process on one GPU)."""
        self._guard()
        assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
        T, H = x.shape
        assert H == self.H and T <= self.cap
        K = self.K
        if lay is None:
            lay = out.layout if out is not None else self.layout(topk_idx)
        if out is None:
            n_cap = n_cap if n_cap is not None else self.R * self.cap * min(K, self.E // self.R)
            a_cap = a_cap if a_cap is not None else self.R * self.cap
            dev = x.device
            if quant:
                recv_x = torch.empty(n_cap, H, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
                recv_s = torch.empty(n_cap, H // 128, dtype=torch.float32, device=dev)
            else:
                recv_x = torch.empty(n_cap, H, dtype=torch.bfloat16, device=dev)
                recv_s = None
            out = DispatchResult(
                recv_x, recv_s, torch.empty(n_cap, 3, dtype=torch.int32, device=dev),
                torch.empty(self.E, dtype=torch.int32, device=dev),
                torch.empty(self.E // self.R, dtype=torch.int64, device=dev),
                torch.empty(a_cap, 2 * K + 2, dtype=torch.int32, device=dev),
                torch.zeros(4 + MAX_RANKS, dtype=torch.int32, device=dev), lay, topk_idx, topk_weights, T, quant)
        p = _DispatchParams()
        p.R, p.rank, p.E, p.K, p.H, p.cap, p.quant, p.T = self.R, self.rank, self.E, K, H, self.cap, int(quant), T
        p.n_cap, p.a_cap = out.recv_x.shape[0], out.recv_meta.shape[0]
        p.num_ctas, p.phase_mask = self.num_ctas, phase_mask
        for i, pp in enumerate(self.heap.peer_ptrs):
            p.peers[i] = pp
        p.x, p.topk_idx = x.data_ptr(), topk_idx.data_ptr()
        p.topk_w = topk_weights.data_ptr() if topk_weights is not None else None
        p.send_idx, p.rank_slot = lay.send_token_idx.data_ptr(), lay.rank_slot.data_ptr()
        p.num_per_expert, p.num_per_rank = lay.num_tokens_per_expert.data_ptr(), lay.num_tokens_per_rank.data_ptr()
        p.recv_x = out.recv_x.data_ptr()
        p.recv_scales = out.recv_scales.data_ptr() if out.recv_scales is not None else None
        p.expand_idx, p.recv_count = out.expand_idx.data_ptr(), out.recv_count.data_ptr()
        p.recv_per_expert, p.recv_meta = out.recv_tokens_per_expert.data_ptr(), out.recv_meta.data_ptr()
        p.counts_dev, p.counts_host = out.counts.data_ptr(), self.mirror.dev_ptr
        p.ctrl, p.status = self.ctrl.data_ptr(), self.status.data_ptr()
        p.diag = self.diag_dispatch.data_ptr() if self.diagnose else None
        rc = self.lib.umdk_ep_dispatch(ctypes.byref(p), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_ep_dispatch failed: {rc}")
        if sync_counts and (phase_mask & 2):
            torch.cuda.current_stream().synchronize()
            check_status(self.status, "ep_dispatch", owner=self)
            out.num_recv = int(self.mirror.host[0])
        return out

    @_trace.traced("umdk.ep.combine")
    def combine(self, y: torch.Tensor, disp: DispatchResult, apply_weights: bool = True, phase_mask: int = 3,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Per-rank pre-reduced combine: out[t] = sum over ranks of (sum_k w[t,k] * y_row(t,k))."""
        self._guard()
        assert y.is_cuda and y.dtype == torch.bfloat16 and y.is_contiguous() and y.shape[1] == self.H
        T = disp.num_tokens
        if out is None:
            out = torch.empty(T, self.H, dtype=torch.bfloat16, device=y.device)
        p = _CombineParams()
        p.R, p.rank, p.E, p.K, p.H, p.cap, p.T = self.R, self.rank, self.E, self.K, self.H, self.cap, T
        p.mode, p.apply_weights, p.n_rows = 0, int(apply_weights), 0
        p.num_ctas, p.phase_mask = self.num_ctas, phase_mask
        for i, pp in enumerate(self.heap.peer_ptrs):
            p.peers[i] = pp
        p.y, p.recv_meta, p.counts_dev = y.data_ptr(), disp.recv_meta.data_ptr(), disp.counts.data_ptr()
        p.in_rank = disp.layout.is_token_in_rank.data_ptr()
        p.out, p.ctrl, p.status = out.data_ptr(), self.ctrl.data_ptr(), self.status.data_ptr()
        p.diag = self.diag_combine.data_ptr() if self.diagnose else None
        rc = self.lib.umdk_ep_combine(ctypes.byref(p), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_ep_combine failed: {rc}")
        return out

    @_trace.traced("umdk.ep.combine_rows")
    def combine_rows(self, y: torch.Tensor, src_idx: torch.Tensor, topk_idx: torch.Tensor,
                     topk_weights: torch.Tensor, phase_mask: int = 3, out: Optional[torch.Tensor] = None
                     ) -> torch.Tensor:
        """Row-per-(token,k) combine with the reference's stateless contract (moe_combine_prefill)."""
        self._guard()
        T = topk_idx.shape[0]
        if out is None:
            out = torch.empty(T, self.H, dtype=torch.bfloat16, device=y.device)
        p = _CombineParams()
        p.R, p.rank, p.E, p.K, p.H, p.cap, p.T = self.R, self.rank, self.E, self.K, self.H, self.cap, T
        p.mode, p.apply_weights, p.n_rows = 1, 1, y.shape[0]
        p.num_ctas, p.phase_mask = self.num_ctas, phase_mask
        for i, pp in enumerate(self.heap.peer_ptrs):
            p.peers[i] = pp
        p.y, p.src_idx = y.data_ptr(), src_idx.data_ptr()
        p.topk_idx, p.topk_w = topk_idx.data_ptr(), topk_weights.data_ptr()
        p.out, p.ctrl, p.status = out.data_ptr(), self.ctrl.data_ptr(), self.status.data_ptr()
        p.diag = self.diag_combine.data_ptr() if self.diagnose else None
        rc = self.lib.umdk_ep_combine(ctypes.byref(p), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_ep_combine failed: {rc}")
        return out

    def check(self, what: str = "ep"):
        check_status(self.status, what, owner=self)
