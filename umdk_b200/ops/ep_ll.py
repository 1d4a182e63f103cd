"""Low-latency (decode) expert-parallel MoE layer on the GPU: dispatch -> grouped fp8 GEMM1 + SwiGLU + re-quant ->
grouped fp8 GEMM2 whose epilogue stores rows into the token owners' combine buffers -> top-k weighted reduction.

One launch per call (on the caller's stream, capturable in a CUDA graph): ``moe_fused`` runs the dispatch as its
prologue (routing layout in shared memory, count all-gather, fp8 1x128 quantisation, direct push into the destination
slab rows), waits for the arrival flags, then gate/up projection + SwiGLU + fp8 re-quantisation, down projection with
the combine-send epilogue, completion flags and the owner-side weighted reduction. The stages also exist as separate
launches (``dispatch`` = ep_ll_dispatch, ``fuse_dispatch=False``; ``fused=False`` = moe_gemm mode 0 then mode 2), which
is how tests drive several emulated ranks on one GPU and what ``Buffer.low_latency_dispatch`` uses.
The shared expert (if any) runs through the same GEMM kernels on the locally quantised tokens.

Mirrors the contract of the reference's ``fused_deep_moe`` (src/cam/comm_operator/pybind/fused_deep_moe.cpp:30-83;
doc/en/cam/CAM API Guide.md:150-226): returns (combine_x, share_output, expert_token_nums) with the shared expert's
output returned separately, ``expert_ids == -1`` skipped.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import _native
from ..parallel.symm import SymmetricHeap
from . import moe_gemm
from .ep import Recoverable, check_status, layout as ep_layout
from ..utils import trace as _trace

MAX_RANKS = 32


class _LLLayout(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in
                ("cnt", "cnt_flag", "data_flag", "comb_flag", "slab_x", "slab_s", "slab_meta", "comb_buf", "total")] + \
               [("n_cap", ctypes.c_int), ("exp_cnt", ctypes.c_uint64)]


class _LLDispatchParams(ctypes.Structure):
    _fields_ = [
        ("R", ctypes.c_int), ("rank", ctypes.c_int), ("E", ctypes.c_int), ("K", ctypes.c_int), ("H", ctypes.c_int),
        ("T_cap", ctypes.c_int), ("T", ctypes.c_int), ("num_ctas", ctypes.c_int), ("phase_mask", ctypes.c_int),
        ("peers", ctypes.c_void_p * MAX_RANKS),
        ("x", ctypes.c_void_p), ("topk_idx", ctypes.c_void_p), ("send_idx", ctypes.c_void_p),
        ("num_per_expert", ctypes.c_void_p), ("group_off", ctypes.c_void_p), ("recv_per_expert", ctypes.c_void_p),
        ("ctrl", ctypes.c_void_p), ("status", ctypes.c_void_p),
    ]


class _LLCombineParams(ctypes.Structure):
    _fields_ = [
        ("R", ctypes.c_int), ("rank", ctypes.c_int), ("E", ctypes.c_int), ("K", ctypes.c_int), ("H", ctypes.c_int),
        ("T_cap", ctypes.c_int), ("T", ctypes.c_int), ("num_ctas", ctypes.c_int), ("phase_mask", ctypes.c_int),
        ("peers", ctypes.c_void_p * MAX_RANKS),
        ("y", ctypes.c_void_p), ("group_off", ctypes.c_void_p), ("topk_idx", ctypes.c_void_p),
        ("topk_w", ctypes.c_void_p), ("out", ctypes.c_void_p), ("ctrl", ctypes.c_void_p), ("status", ctypes.c_void_p),
    ]


class _MoeFusedParams(ctypes.Structure):
    _fields_ = [
        ("G", ctypes.c_int), ("F", ctypes.c_int), ("H", ctypes.c_int), ("n_rows_cap", ctypes.c_int),
        ("max_ctas", ctypes.c_int), ("w_tiled", ctypes.c_int),
        ("w1", ctypes.c_void_p), ("w1s", ctypes.c_void_p), ("w2", ctypes.c_void_p), ("w2s", ctypes.c_void_p),
        ("x", ctypes.c_void_p), ("xs", ctypes.c_void_p), ("group_off", ctypes.c_void_p),
        ("hq", ctypes.c_void_p), ("hs", ctypes.c_void_p), ("tile_done", ctypes.c_void_p),
        ("wait_flags", ctypes.c_void_p), ("wait_n", ctypes.c_int),
        ("R", ctypes.c_int), ("rank", ctypes.c_int), ("T", ctypes.c_int), ("Kt", ctypes.c_int),
        ("T_cap", ctypes.c_int),
        ("peers", ctypes.c_void_p * MAX_RANKS),
        ("comb_buf_off", ctypes.c_uint64), ("comb_flag_off", ctypes.c_uint64),
        ("row_meta", ctypes.c_void_p), ("topk_idx", ctypes.c_void_p), ("topk_w", ctypes.c_void_p),
        ("out", ctypes.c_void_p), ("share_out", ctypes.c_void_p), ("ctrl", ctypes.c_void_p),
        ("phase_mask", ctypes.c_int), ("status", ctypes.c_void_p), ("diag", ctypes.c_void_p),
        ("disp_x", ctypes.c_void_p), ("E", ctypes.c_int), ("recv_per_expert", ctypes.c_void_p),
        ("group_off_out", ctypes.c_void_p),
    ]


def ll_layout(R: int, E: int, K: int, H: int, T_cap: int) -> _LLLayout:
    lib = _native.cam()
    lay = _LLLayout()
    rc = lib.umdk_ep_ll_layout(R, E, K, H, T_cap, ctypes.byref(lay))
    if rc != 0:
        raise ValueError(f"unsupported low-latency geometry R={R} E={E} K={K} H={H} T_cap={T_cap}")
    return lay


def quant_fp8_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [T, H] -> (fp8 e4m3 [T, H], fp32 scales [T, H/128]) with the hand-written kernel."""
    lib = _native.cam()
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
    T, H = x.shape
    q = torch.empty(T, H, dtype=torch.uint8, device=x.device).view(torch.float8_e4m3fn)
    s = torch.empty(T, H // 128, dtype=torch.float32, device=x.device)
    rc = lib.umdk_quant_fp8_1x128(_native.ptr(x), T, H, _native.ptr(q), _native.ptr(s), _native.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"umdk_quant_fp8_1x128 failed: {rc}")
    return q, s


@dataclass
class ExpertWeights:
    """fp8 e4m3 expert weights with 128x128 block scales. w1: [G, 2F, H] (gate rows first), w2: [G, H, F]."""
    w1q: torch.Tensor
    w1s: torch.Tensor
    w2q: torch.Tensor
    w2s: torch.Tensor
    tiled: bool = False   # w1q / w2q hold the tile-major repacking (only the fused kernel reads it)

    def to_tiled(self) -> "ExpertWeights":
        """Repacks the fp8 weights so that every 128 x 128-byte tile a k-block needs is one contiguous chunk
        (w1: [G, F/128, H/128, 256, 128] with the gate rows of the tile followed by its up rows;
        w2: [G, H/128, F/128, 128, 128]). Done once at load time; the fused kernel then streams 32 KB / 16 KB
        sequential pieces instead of 128-byte pieces a row apart. Scales are shared with the original."""
        if self.tiled:
            return self
        G, F2, H = self.w1q.shape
        F = F2 // 2
        w1 = self.w1q.view(torch.uint8).view(G, 2, F // 128, 128, H // 128, 128)
        w1t = w1.permute(0, 2, 4, 1, 3, 5).contiguous().view(G, F // 128, H // 128, 256, 128)
        w2 = self.w2q.view(torch.uint8).view(G, H // 128, 128, F // 128, 128)
        w2t = w2.permute(0, 1, 3, 2, 4).contiguous()
        return ExpertWeights(w1t.view(torch.float8_e4m3fn), self.w1s, w2t.view(torch.float8_e4m3fn), self.w2s, True)

    def to_row_major(self) -> "ExpertWeights":
        """Inverse of ``to_tiled`` (w1: [G, 2F, H], w2: [G, H, F])."""
        if not self.tiled:
            return self
        G, nt, kb = self.w1q.shape[:3]
        w1 = self.w1q.view(torch.uint8).view(G, nt, kb, 2, 128, 128).permute(0, 3, 1, 4, 2, 5).contiguous()
        w2 = self.w2q.view(torch.uint8).permute(0, 1, 3, 2, 4).contiguous()
        return ExpertWeights(w1.view(G, 2 * nt * 128, kb * 128).view(torch.float8_e4m3fn), self.w1s,
                             w2.view(G, self.w2q.shape[1] * 128, self.w2q.shape[2] * 128).view(torch.float8_e4m3fn),
                             self.w2s, False)

    @property
    def num_local_experts(self) -> int:
        return self.w1q.shape[0]

    @staticmethod
    def with_shared(experts: "ExpertWeights", shared: "ExpertWeights") -> "ExpertWeights":
        """Local experts followed by the shared expert as one more local expert (the layout ``fold_shared`` wants)."""
        def cat8(a, b):
            return torch.cat((a.view(torch.uint8), b.view(torch.uint8))).contiguous().view(torch.float8_e4m3fn)
        return ExpertWeights(cat8(experts.w1q, shared.w1q), torch.cat((experts.w1s, shared.w1s)).contiguous(),
                             cat8(experts.w2q, shared.w2q), torch.cat((experts.w2s, shared.w2s)).contiguous())


class EpLowLatency(Recoverable):
    """Per-rank state of the low-latency MoE path at a fixed geometry."""

    _epoch_words = {"ctrl": (0,)}
    _zero_between_calls = ("layout_bar", "tile_done", "exp_cnt")

    def __init__(self, heap: SymmetricHeap, num_experts: int, top_k: int, hidden: int, ffn: int, t_cap: int,
                 dispatch_ctas: int = 32, gemm_ctas: int = 0, fold_shared: bool = False):
        """``fold_shared``: the shared expert runs inside the routed pipeline as one more local expert that every
        token of this rank is sent to with weight 1 (so its tiles are scheduled with all the others instead of a
        separate under-filled launch). The geometry then has num_experts + R experts and top_k + 1 slots; ``moe`` takes
        weights built by ``ExpertWeights.with_shared`` and still returns the shared output separately. Use
        ``heap_bytes(..., fold_shared=True)`` to size the heap."""
        self.lib = _native.cam()
        self.heap = heap
        self.R, self.rank = heap.world, heap.rank
        self.fold = fold_shared
        self.E_user, self.K_user = num_experts, top_k
        if fold_shared:
            num_experts, top_k = num_experts + heap.world, top_k + 1
        self.E, self.K, self.H, self.F, self.T_cap = num_experts, top_k, hidden, ffn, t_cap
        self.E_local = num_experts // self.R
        self.lay = ll_layout(self.R, num_experts, top_k, hidden, t_cap)
        if self.lay.total > heap.nbytes:
            raise ValueError(f"symmetric heap too small: need {self.lay.total}, have {heap.nbytes}")
        self.n_cap = self.lay.n_cap
        dev = torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        self.ctrl = torch.zeros(16, dtype=torch.int32, device=dev)
        # diagnose mode: the fused kernel stamps its stages with the global timer (see timeline_us)
        self.diagnose = False
        self.diag_fused = torch.zeros(6, dtype=torch.int64, device=dev)
        self.inline_layout = True   # False: run the layout kernel as a launch of its own before every dispatch
        self.fuse_dispatch = True   # moe(): the dispatch runs inside the fused kernel (one launch per layer)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self.layout_bar = torch.zeros(2, dtype=torch.int32, device=dev)
        self.layout_scratch = torch.empty(((t_cap + 31) // 32) * (num_experts + self.R), dtype=torch.int32, device=dev)
        self.group_off = torch.zeros(self.E_local + 1, dtype=torch.int32, device=dev)
        self.recv_per_expert = torch.zeros(self.E_local, dtype=torch.int64, device=dev)
        self.hq = torch.empty(self.n_cap, ffn, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        self.hs = torch.empty(self.n_cap, ffn // 128, dtype=torch.float32, device=dev)
        self.dispatch_ctas, self.gemm_ctas = dispatch_ctas, gemm_ctas
        # per-token-tile completion counters of the fused kernel (zero between calls; the kernel resets them)
        self.tile_done = torch.zeros(self.n_cap // 64 + self.E_local + 1, dtype=torch.int32, device=dev)
        # shared-expert scratch
        self.sh_off = torch.tensor([0, 0], dtype=torch.int32, device=dev)
        self.sh_hq = torch.empty(t_cap, ffn, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        self.sh_hs = torch.empty(t_cap, ffn // 128, dtype=torch.float32, device=dev)
        # per-expert arrival words in this rank's heap (added to by every sender's dispatch, zeroed by whatever ends
        # the call here); part of what reset() clears
        from ..utils.rawtensor import from_ptr
        self.exp_cnt = from_ptr(self._local(self.lay.exp_cnt), (self.E_local,), torch.int32, dev)

    @staticmethod
    def heap_bytes(R: int, E: int, K: int, H: int, T_cap: int, fold_shared: bool = False) -> int:
        if fold_shared:
            E, K = E + R, K + 1
        return int(ll_layout(R, E, K, H, T_cap).total)

    def fold_routing(self, topk_idx: torch.Tensor, topk_w: torch.Tensor):
        """[T, K] routing over the user's experts -> [T, K + 1] routing over the folded expert numbering (every rank
        has one more local expert, the shared one, which each of its own tokens selects with weight 1)."""
        el = self.E_user // self.R
        T = topk_idx.shape[0]
        idx = torch.empty(T, self.K, dtype=torch.int64, device=topk_idx.device)
        w = torch.empty(T, self.K, dtype=torch.float32, device=topk_idx.device)
        idx[:, :self.K_user] = torch.where(topk_idx >= 0, topk_idx + torch.div(topk_idx, el, rounding_mode="floor"),
                                           topk_idx)
        idx[:, self.K_user] = self.rank * (el + 1) + el
        w[:, :self.K_user] = topk_w
        w[:, self.K_user] = 1.0
        return idx, w

    # -- views into this rank's own heap -------------------------------------------------------------------------
    def _local(self, off: int) -> int:
        return self.heap.local_ptr + off

    def slab_views(self):
        """(slab_x fp8 [n_cap, H], slab_s fp32 [n_cap, H/128], slab_meta int32 [n_cap, 2]) as torch tensors."""
        from ..utils.rawtensor import from_ptr
        x = from_ptr(self._local(self.lay.slab_x), (self.n_cap, self.H), torch.uint8, self.device).view(
            torch.float8_e4m3fn)
        s = from_ptr(self._local(self.lay.slab_s), (self.n_cap, self.H // 128), torch.float32, self.device)
        m = from_ptr(self._local(self.lay.slab_meta), (self.n_cap, 2), torch.int32, self.device)
        return x, s, m

    # -- kernels -------------------------------------------------------------------------------------------------
    @_trace.traced("umdk.ep_ll.dispatch")
    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, phase_mask: int = 3, lay=None):
        self._guard()
        assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and topk_idx.dtype == torch.int64
        T = x.shape[0]
        assert T <= self.T_cap and x.shape[1] == self.H
        # decode-sized inputs: the dispatch kernel derives bucket positions and sizes itself (no layout launch)
        inline = lay is None and self.inline_layout and T <= 2048 and self.E <= 1024 and \
            2 * (((T + 31) // 32) * self.E + 2 * T * self.K) <= 160 * 1024
        if lay is None and not inline:
            lay = ep_layout(topk_idx, self.E, self.R, self.layout_scratch, self.layout_bar, self.status)
        p = _LLDispatchParams()
        p.R, p.rank, p.E, p.K, p.H, p.T_cap, p.T = self.R, self.rank, self.E, self.K, self.H, self.T_cap, T
        p.num_ctas, p.phase_mask = self.dispatch_ctas, phase_mask
        for i, pp in enumerate(self.heap.peer_ptrs):
            p.peers[i] = pp
        p.x, p.topk_idx = x.data_ptr(), topk_idx.data_ptr()
        if lay is not None:
            p.send_idx, p.num_per_expert = lay.send_token_idx.data_ptr(), lay.num_tokens_per_expert.data_ptr()
        else:
            p.send_idx = p.num_per_expert = None
        p.group_off, p.recv_per_expert = self.group_off.data_ptr(), self.recv_per_expert.data_ptr()
        p.ctrl, p.status = self.ctrl.data_ptr(), self.status.data_ptr()
        rc = self.lib.umdk_ep_ll_dispatch(ctypes.byref(p), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_ep_ll_dispatch failed: {rc}")
        return lay

    @_trace.traced("umdk.ep_ll.combine")
    def combine(self, y: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor,
                out: Optional[torch.Tensor] = None, phase_mask: int = 3, num_ctas: int = 0) -> torch.Tensor:
        """Low-latency combine of caller-computed expert outputs ``y`` [>= rows, H] bf16 (slab row order of the last
        ``dispatch``): rows return to their owners over NVLink, flags, weighted sum - one launch, no host
        synchronisation (the row count is read on the device). Ends the call that ``dispatch`` began."""
        self._guard()
        assert y.is_cuda and y.dtype == torch.bfloat16 and y.is_contiguous() and y.shape[1] == self.H
        assert y.shape[0] >= min(self.n_cap, y.shape[0]) and topk_idx.dtype == torch.int64 and topk_idx.is_contiguous()
        T = topk_idx.shape[0]
        if out is None:
            out = torch.empty(T, self.H, dtype=torch.bfloat16, device=y.device)
        p = _LLCombineParams()
        p.R, p.rank, p.E, p.K, p.H, p.T_cap, p.T = self.R, self.rank, self.E, self.K, self.H, self.T_cap, T
        p.num_ctas, p.phase_mask = num_ctas, phase_mask
        for i, pp in enumerate(self.heap.peer_ptrs):
            p.peers[i] = pp
        p.y, p.group_off = y.data_ptr(), self.group_off.data_ptr()
        p.topk_idx, p.topk_w, p.out = topk_idx.data_ptr(), topk_w.data_ptr(), out.data_ptr()
        p.ctrl, p.status = self.ctrl.data_ptr(), self.status.data_ptr()
        rc = self.lib.umdk_ep_ll_combine(ctypes.byref(p), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_ep_ll_combine failed: {rc}")
        return out

    def _gemm1(self, w: ExpertWeights):
        p = moe_gemm.MoeGemmParams()
        p.mode, p.G, p.Nout, p.K = 0, self.E_local, self.F, self.H
        p.n_rows_cap, p.max_ctas = self.n_cap, self.gemm_ctas
        p.w, p.ws = w.w1q.data_ptr(), w.w1s.data_ptr()
        p.x, p.xs = self._local(self.lay.slab_x), self._local(self.lay.slab_s)
        p.group_off = self.group_off.data_ptr()
        p.hq, p.hs = self.hq.data_ptr(), self.hs.data_ptr()
        p.wait_flags[0] = p.wait_flags[1] = self._local(self.lay.data_flag)
        p.wait_n, p.epoch_ptr = self.R, self.ctrl.data_ptr()
        p.status = self.status.data_ptr()
        rc = self.lib.umdk_moe_gemm(ctypes.byref(p), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_moe_gemm(mode 0) failed: {rc}")

    def _gemm2_combine(self, w: ExpertWeights, topk_idx, topk_w, out, phase_mask: int = 3):
        T = topk_idx.shape[0]
        p = moe_gemm.MoeGemmParams()
        p.mode, p.G, p.Nout, p.K = 2, self.E_local, self.H, self.F
        p.n_rows_cap, p.max_ctas = self.n_cap, self.gemm_ctas
        p.w, p.ws = w.w2q.data_ptr(), w.w2s.data_ptr()
        p.x, p.xs = self.hq.data_ptr(), self.hs.data_ptr()
        p.group_off = self.group_off.data_ptr()
        p.epoch_ptr = self.ctrl.data_ptr()
        p.R, p.rank, p.T, p.Kt, p.T_cap = self.R, self.rank, T, self.K, self.T_cap
        for i, pp in enumerate(self.heap.peer_ptrs):
            p.peers[i] = pp
        p.comb_buf_off[0] = p.comb_buf_off[1] = self.lay.comb_buf
        p.comb_flag_off[0] = p.comb_flag_off[1] = self.lay.comb_flag
        p.row_meta = self._local(self.lay.slab_meta)
        p.topk_idx, p.topk_w, p.out = topk_idx.data_ptr(), topk_w.data_ptr(), out.data_ptr()
        p.ctrl = self.ctrl.data_ptr()
        p.status = self.status.data_ptr()
        p.phase_mask = phase_mask
        rc = self.lib.umdk_moe_gemm(ctypes.byref(p), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_moe_gemm(mode 2) failed: {rc}")

    def timeline_reset(self) -> None:
        """Arms the stage stamps of the next fused call (diagnose mode)."""
        self.diag_fused.zero_()
        self.diag_fused[0] = torch.iinfo(torch.int64).max

    @staticmethod
    def timeline_names():
        return ("rows_ready", "phase1", "phase2", "peers_done", "end")

    def timeline_us(self) -> dict:
        """Stages of the last fused kernel in microseconds since its first CTA started, each taken at the LAST CTA to
        get there: rows_ready (dispatched rows arrived), phase1 (GEMM1 + SwiGLU + requant), phase2 (GEMM2 + combine
        send), peers_done (every peer's combine flag seen), end."""
        d = self.diag_fused.tolist()
        names = ("rows_ready", "phase1", "phase2", "peers_done", "end")
        return {n: (d[i + 1] - d[0]) / 1e3 for i, n in enumerate(names)}

    def can_fuse_dispatch(self, T: int) -> bool:
        """The in-kernel dispatch derives the layout in shared memory (16-bit tables inside the operand ring)."""
        return T <= 2048 and self.E <= 1024 and \
            64 + 16 * self.E + 2 * (((T + 31) // 32) * self.E + 2 * T * self.K) + 3072 <= 160 * 1024

    def _fused(self, w: ExpertWeights, topk_idx, topk_w, out, phase_mask: int = 3, share_out=None, x=None):
        """GEMM1 + SwiGLU + re-quant + GEMM2 + combine-send + weighted reduction in ONE persistent launch
        (csrc/cam/moe_fused.cu). With ``x`` (this rank's bf16 tokens) the dispatch runs inside the same launch:
        phase_mask bit 2 publishes the counts, bit 3 pushes the rows, bit 0 / bit 1 as without it (15 = everything)."""
        self._guard()
        p = _MoeFusedParams()
        if x is not None:
            assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape == (topk_idx.shape[0], self.H)
            assert self.can_fuse_dispatch(x.shape[0])
            p.disp_x, p.E = x.data_ptr(), self.E
            p.recv_per_expert, p.group_off_out = self.recv_per_expert.data_ptr(), self.group_off.data_ptr()
        p.G, p.F, p.H, p.n_rows_cap, p.max_ctas = self.E_local, self.F, self.H, self.n_cap, self.gemm_ctas
        p.w_tiled = 1 if w.tiled else 0
        p.w1, p.w1s, p.w2, p.w2s = w.w1q.data_ptr(), w.w1s.data_ptr(), w.w2q.data_ptr(), w.w2s.data_ptr()
        p.x, p.xs = self._local(self.lay.slab_x), self._local(self.lay.slab_s)
        p.group_off = self.group_off.data_ptr()
        p.hq, p.hs, p.tile_done = self.hq.data_ptr(), self.hs.data_ptr(), self.tile_done.data_ptr()
        p.wait_flags, p.wait_n = self._local(self.lay.data_flag), self.R
        p.R, p.rank, p.T, p.Kt, p.T_cap = self.R, self.rank, topk_idx.shape[0], self.K, self.T_cap
        for i, pp in enumerate(self.heap.peer_ptrs):
            p.peers[i] = pp
        p.comb_buf_off, p.comb_flag_off = self.lay.comb_buf, self.lay.comb_flag
        p.row_meta = self._local(self.lay.slab_meta)
        p.topk_idx, p.topk_w, p.out = topk_idx.data_ptr(), topk_w.data_ptr(), out.data_ptr()
        p.share_out = share_out.data_ptr() if share_out is not None else None
        p.ctrl, p.phase_mask, p.status = self.ctrl.data_ptr(), phase_mask, self.status.data_ptr()
        p.diag = self.diag_fused.data_ptr() if self.diagnose else None
        rc = self.lib.umdk_moe_fused(ctypes.byref(p), _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"umdk_moe_fused failed: {rc}")

    def shared_expert(self, x: torch.Tensor, w: ExpertWeights, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Dense SwiGLU FFN of the shared expert on this rank's own tokens (fp8 block-scaled, same GEMM kernels)."""
        T = x.shape[0]
        xq, xs = quant_fp8_1x128(x)
        self.sh_off[1] = T
        moe_gemm.gemm1_swiglu_quant(xq, xs, self.sh_off, w.w1q, w.w1s, self.status, self.sh_hq[:T], self.sh_hs[:T],
                                    max_ctas=self.gemm_ctas)
        return moe_gemm.gemm2(self.sh_hq[:T], self.sh_hs[:T], self.sh_off, w.w2q, w.w2s, self.status, y=out,
                              max_ctas=self.gemm_ctas)

    @_trace.traced("umdk.ep_ll.moe")
    def moe(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, w: ExpertWeights,
            shared: Optional[ExpertWeights] = None, out: Optional[torch.Tensor] = None, fused: bool = True,
            prefolded: bool = False):
        """Full layer: returns (combine_x [T, H] bf16, share_output or None, expert_token_nums [E_local] int64).
        ``fused`` runs both expert GEMMs and the combine as one persistent kernel; otherwise as two launches.
        ``prefolded`` (fold_shared only): ``topk_idx`` / ``topk_w`` are already [T, K + 1] in the folded numbering
        (what ``fold_routing`` or ops.glue.router_topk(fold_el=...) produce)."""
        T = x.shape[0]
        if out is None:
            out = torch.empty(T, self.H, dtype=torch.bfloat16, device=x.device)
        if self.fold:
            assert shared is None and fused and w.w1q.shape[0] == self.E_local, \
                "fold_shared: pass ExpertWeights.with_shared(experts, shared) as w"
            idx, wts = (topk_idx, topk_w) if prefolded else self.fold_routing(topk_idx, topk_w)
            assert idx.shape[1] == self.K
            share_out = torch.empty(T, self.H, dtype=torch.bfloat16, device=x.device)
            if self.fuse_dispatch and self.inline_layout and self.can_fuse_dispatch(T):
                self._fused(w, idx, wts, out, share_out=share_out, x=x, phase_mask=15)
            else:
                self.dispatch(x, idx)
                self._fused(w, idx, wts, out, share_out=share_out)
            return out, share_out, self.recv_per_expert[:self.E_local - 1]
        one_launch = fused and self.fuse_dispatch and self.inline_layout and self.can_fuse_dispatch(T)
        if not one_launch:
            self.dispatch(x, topk_idx)
        share_out = self.shared_expert(x, shared) if shared is not None else None
        if one_launch:
            self._fused(w, topk_idx, topk_w, out, x=x, phase_mask=15)
        elif fused:
            self._fused(w, topk_idx, topk_w, out)
        else:
            assert not w.tiled, "the two-launch path reads row-major weights"
            self._gemm1(w)
            self._gemm2_combine(w, topk_idx, topk_w, out)
        return out, share_out, self.recv_per_expert

    @_trace.traced("umdk.ep_ll.capture")
    def capture(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, w: ExpertWeights,
                shared: Optional[ExpertWeights] = None, out: Optional[torch.Tensor] = None):
        """Records the whole layer (layout, dispatch, fused expert kernel) into a CUDA graph and returns
        ``(graph, (combine_x, share_output, expert_token_nums))``. ``graph.replay()`` then re-runs it on the CURRENT
        contents of ``x`` / ``topk_idx`` / ``topk_w`` with one launch from the host, which takes the Python and
        driver launch costs of the three kernels off the critical path of a decode step. All epoch / flag state
        lives in device memory, so replays chain like ordinary calls; every rank must replay the same number of
        times. Call ``torch.cuda.synchronize()`` (and a barrier across ranks) before capturing."""
        T = x.shape[0]
        if out is None:
            out = torch.empty(T, self.H, dtype=torch.bfloat16, device=x.device)
        self.moe(x, topk_idx, topk_w, w, shared, out=out)   # first call outside the capture: attribute setup, caches
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            res = self.moe(x, topk_idx, topk_w, w, shared, out=out)
        return g, res

    def check(self, what: str = "ep_ll"):
        check_status(self.status, what, owner=self)
