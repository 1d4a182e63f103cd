"""DeepEP-style communication buffer for expert-parallel MoE: `get_dispatch_layout`, `dispatch`, `combine`,
`low_latency_dispatch`, `low_latency_combine` and the fully fused `fused_moe`.

The reference replaces DeepEP's `Buffer` methods with its torch ops one for one (skills/deepep-to-cam-converter/
SKILL.md:83-90; references/cam_dispatch_and_combine_a3.md:200-282); this class offers the same call shapes on top of
the B200 kernels (CUDA tensors, NCCL-bootstrapped symmetric heap) and on top of gloo all-to-all for CPU tensors.

Differences from DeepEP that callers see:
  * `dispatch` returns rows already grouped by local expert (expert-major, then source rank), one row per
    (token, k) - the layout a grouped GEMM wants and the layout of the reference's `recv_x`. `recv_topk_idx` is the
    local expert of each row, `recv_topk_weights` the routing weight of each row.
  * fp8 payloads are e4m3 with one fp32 scale per 1x128 block: `recv_x` is then the tuple `(x_fp8, scales)`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple, Union

import torch
import torch.distributed as dist

from .ops import cpu_dist
from .ops import reference as ref
from .utils import trace as _trace


class EventOverlap:
    """CUDA event handle returned by the asynchronous forms of the Buffer methods."""

    def __init__(self, event: Optional["torch.cuda.Event"] = None):
        self.event = event

    def current_stream_wait(self):
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.current_stream_wait()


@dataclass
class Config:
    """Tuning knobs (DeepEP's `deep_ep.Config` analogue): number of CTAs used by the communication kernels."""
    num_sms: int = 0


@dataclass
class DispatchHandle:
    backend: str
    topk_idx: torch.Tensor
    topk_weights: Optional[torch.Tensor]
    num_tokens: int
    gpu: object = None   # ops.ep.DispatchResult
    cpu: object = None   # ops.cpu_dist.CpuDispatchResult


class Buffer:
    num_sms = 0

    def __init__(self, group: Optional[dist.ProcessGroup] = None, num_nvl_bytes: int = 0, num_rdma_bytes: int = 0,
                 low_latency_mode: bool = False, num_experts: Optional[int] = None, hidden: Optional[int] = None,
                 top_k: Optional[int] = None, max_tokens_per_rank: int = 4096, ffn_hidden: Optional[int] = None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.group_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.low_latency_mode = low_latency_mode
        self.num_nvl_bytes, self.num_rdma_bytes = num_nvl_bytes, num_rdma_bytes
        self.max_tokens_per_rank = max_tokens_per_rank
        self._geom_hint = (num_experts, top_k, hidden, ffn_hidden)
        self._normal = {}   # (E, K, H, cap) -> (heap, EpNormal)
        self._ll = {}       # (E, K, H, F, cap) -> (heap, EpLowLatency)

    # ---- sizing helpers (DeepEP API parity) ----------------------------------------------------------------------
    @staticmethod
    def get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int,
                                       num_experts: int, top_k: int = 8) -> int:
        from .ops.ep_ll import EpLowLatency
        return EpLowLatency.heap_bytes(num_ranks, num_experts, top_k, hidden, num_max_dispatch_tokens_per_rank)

    @staticmethod
    def get_normal_size_hint(max_tokens_per_rank: int, hidden: int, num_ranks: int, num_experts: int,
                             top_k: int = 8) -> int:
        from .ops.ep import EpNormal
        return EpNormal.heap_bytes(num_ranks, num_experts, top_k, hidden, max_tokens_per_rank)

    @staticmethod
    def set_num_sms(n: int):
        Buffer.num_sms = n

    # ---- state -----------------------------------------------------------------------------------------------
    def _normal_state(self, E: int, K: int, H: int, T: int):
        from .ops.ep import EpNormal
        from .parallel.symm import SymmetricHeap
        cap = max(self.max_tokens_per_rank, T)
        key = (E, K, H, cap)
        if key not in self._normal:
            nbytes = EpNormal.heap_bytes(self.group_size, E, K, H, cap)
            heap = SymmetricHeap(nbytes, self.group) if self.group_size > 1 else SymmetricHeap(nbytes)
            self._normal[key] = (heap, EpNormal(heap, E, K, H, cap, num_ctas=Buffer.num_sms))
        return self._normal[key][1]

    def _ll_state(self, E: int, K: int, H: int, F: int, T: int):
        from .ops.ep_ll import EpLowLatency
        from .parallel.symm import SymmetricHeap
        key = (E, K, H, F, T)
        if key not in self._ll:
            nbytes = EpLowLatency.heap_bytes(self.group_size, E, K, H, T)
            heap = SymmetricHeap(nbytes, self.group) if self.group_size > 1 else SymmetricHeap(nbytes)
            self._ll[key] = (heap, EpLowLatency(heap, E, K, H, F, T))
        return self._ll[key][1]

    def destroy(self):
        for heap, _ in list(self._normal.values()) + list(self._ll.values()):
            heap.close()
        self._normal.clear()
        self._ll.clear()

    # ---- layout ------------------------------------------------------------------------------------------------
    @_trace.traced("umdk.buffer.get_dispatch_layout")
    def get_dispatch_layout(self, topk_idx: torch.Tensor, num_experts: int, previous_event=None,
                            async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """-> (num_tokens_per_rank, num_tokens_per_rdma_rank (None on one box), num_tokens_per_expert,
        is_token_in_rank, event)"""
        if previous_event is not None:
            previous_event.current_stream_wait()
        if topk_idx.is_cuda:
            from .ops.ep import layout
            lay = layout(topk_idx.contiguous(), num_experts, self.group_size)
            ev = EventOverlap(torch.cuda.current_stream().record_event()) if async_finish else EventOverlap()
        else:
            lay = ref.ref_layout(topk_idx, num_experts, self.group_size)
            ev = EventOverlap()
        return lay.num_tokens_per_rank, None, lay.num_tokens_per_expert, lay.is_token_in_rank, ev

    # ---- normal mode ---------------------------------------------------------------------------------------------
    @_trace.traced("umdk.buffer.dispatch")
    def dispatch(self, x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]], handle=None,
                 num_tokens_per_rank=None, num_tokens_per_rdma_rank=None, is_token_in_rank=None,
                 num_tokens_per_expert=None, topk_idx: Optional[torch.Tensor] = None,
                 topk_weights: Optional[torch.Tensor] = None, expert_alignment: int = 1, config: Optional[Config] = None,
                 previous_event=None, async_finish: bool = False, allocate_on_comm_stream: bool = False,
                 use_fp8: bool = True, num_experts: Optional[int] = None, static_shapes: Optional[bool] = None):
        """-> (recv_x, recv_topk_idx, recv_topk_weights, num_recv_tokens_per_expert_list, handle, event)

        With ``static_shapes`` (argument, or the attribute of that name set on the buffer) nothing is read back on
        the host: every result keeps its capacity-bound number of rows, ``num_recv_tokens_per_expert_list`` is the
        device tensor of counts instead of a list, rows past the received ones carry expert id ``-1`` and weight 0.
        That call sequence can be captured in a CUDA graph; the reference's host read of the counts
        (deep_ep/buffer.py: ``num_recv_tokens_per_expert_list``) is what the default form keeps."""
        if previous_event is not None:
            previous_event.current_stream_wait()
        if handle is not None and topk_idx is None:
            topk_idx, topk_weights = handle.topk_idx, handle.topk_weights
        assert topk_idx is not None, "topk_idx (or a handle from an earlier dispatch) is required"
        E = num_experts or (num_tokens_per_expert.numel() if num_tokens_per_expert is not None else self._geom_hint[0])
        assert E is not None, "pass num_experts or num_tokens_per_expert"
        T, K = topk_idx.shape
        el = E // self.group_size
        if x.is_cuda:
            st = self._normal_state(E, K, x.shape[1], T)
            if static_shapes if static_shapes is not None else getattr(self, "static_shapes", False):
                return self._dispatch_static(st, x, topk_idx, topk_weights, use_fp8, el, async_finish)
            out = st.dispatch(x.contiguous(), topk_idx.contiguous(),
                              topk_weights.contiguous() if topk_weights is not None else None, quant=use_fp8,
                              sync_counts=True)
            n = out.num_recv
            per_expert = out.recv_tokens_per_expert.tolist()
            rows_le = torch.repeat_interleave(torch.arange(el, device=x.device),
                                              out.recv_tokens_per_expert.to(x.device))
            # per-row weights travel in the arrival metadata; rebuild them in row order
            recv_w = torch.zeros(n, dtype=torch.float32, device=x.device)
            a = int(out.counts[1].item())
            meta = out.recv_meta[:a]
            rows = meta[:, 2:2 + K].reshape(-1).long()
            wbits = meta[:, 2 + K:2 + 2 * K].reshape(-1).contiguous().view(torch.float32)
            sel = rows >= 0
            recv_w[rows[sel]] = wbits[sel]
            recv_x = (out.recv_x[:n], out.recv_scales[:n]) if use_fp8 else out.recv_x[:n]
            h = DispatchHandle("gpu", topk_idx, topk_weights, T, gpu=out)
            ev = EventOverlap(torch.cuda.current_stream().record_event()) if async_finish else EventOverlap()
            return recv_x, rows_le, recv_w, per_expert, h, ev
        res = cpu_dist.cpu_dispatch(x, topk_idx, topk_weights, E, self.group, quant=use_fp8)
        rows_le = torch.repeat_interleave(torch.arange(el), res.recv_tokens_per_expert)
        recv_x = (res.recv_x, res.recv_scales) if use_fp8 else res.recv_x
        h = DispatchHandle("cpu", topk_idx, topk_weights, T, cpu=res)
        return recv_x, rows_le, res.recv_weights, res.recv_tokens_per_expert.tolist(), h, EventOverlap()

    def _dispatch_static(self, st, x, topk_idx, topk_weights, use_fp8, el, async_finish):
        """Dispatch whose results keep their worst-case sizes; every count stays on the device."""
        T, K = topk_idx.shape
        out = st.dispatch(x.contiguous(), topk_idx.contiguous(),
                          topk_weights.contiguous() if topk_weights is not None else None, quant=use_fp8)
        dev = x.device
        n_cap, a_cap = out.recv_x.shape[0], out.recv_meta.shape[0]
        ends = out.recv_tokens_per_expert.cumsum(0)                       # [E_local] row where each expert ends
        rows_le = torch.searchsorted(ends, torch.arange(n_cap, device=dev), right=True)
        rows_le = torch.where(rows_le < el, rows_le, torch.full_like(rows_le, -1))
        # weights ride in the arrival metadata; rows of arrivals that did not happen are sent to a spare slot
        arrived = (torch.arange(a_cap, device=dev) < out.counts[1]).unsqueeze(1)
        rows = out.recv_meta[:, 2:2 + K].long()
        wbits = out.recv_meta[:, 2 + K:2 + 2 * K].contiguous().view(torch.float32)
        ok = arrived & (rows >= 0) & (rows < n_cap)
        recv_w = torch.zeros(n_cap + 1, dtype=torch.float32, device=dev)
        recv_w.scatter_(0, torch.where(ok, rows, torch.full_like(rows, n_cap)).reshape(-1),
                        torch.where(ok, wbits, torch.zeros_like(wbits)).reshape(-1))
        recv_x = (out.recv_x, out.recv_scales) if use_fp8 else out.recv_x
        h = DispatchHandle("gpu", topk_idx, topk_weights, T, gpu=out)
        ev = EventOverlap(torch.cuda.current_stream().record_event()) if async_finish else EventOverlap()
        return recv_x, rows_le, recv_w[:n_cap], out.recv_tokens_per_expert, h, ev

    @_trace.traced("umdk.buffer.combine")
    def combine(self, x: torch.Tensor, handle: DispatchHandle, topk_weights: Optional[torch.Tensor] = None,
                config: Optional[Config] = None, previous_event=None, async_finish: bool = False,
                allocate_on_comm_stream: bool = False):
        """x: expert outputs in the dispatch row order. -> (combined_x [T, H], combined_topk_weights, event).
        The rows of a token are weighted with the routing weights given at dispatch time (or `topk_weights`)."""
        if previous_event is not None:
            previous_event.current_stream_wait()
        w = topk_weights if topk_weights is not None else handle.topk_weights
        if handle.backend == "gpu":
            d = handle.gpu
            st = self._normal_state(d.recv_count.numel(), handle.topk_idx.shape[1], x.shape[1], handle.num_tokens)
            n_cap = d.recv_x.shape[0]
            if x.shape[0] != n_cap:  # kernel indexes rows < N only; any buffer with >= N rows works
                assert x.shape[0] >= (d.num_recv or 0)
            if topk_weights is not None and topk_weights is not handle.topk_weights:
                n = d.num_recv if d.num_recv is not None else int(d.counts[0].item())
                out = st.combine_rows(x.contiguous(), d.expand_idx[:n].contiguous(), handle.topk_idx.contiguous(),
                                      w.contiguous())
            else:
                out = st.combine(x.contiguous(), d, apply_weights=w is not None)
            ev = EventOverlap(torch.cuda.current_stream().record_event()) if async_finish else EventOverlap()
            return out, w, ev
        c = handle.cpu
        ww = w if w is not None else torch.ones(handle.topk_idx.shape, dtype=torch.float32)
        out = cpu_dist.cpu_combine(x, c.expand_idx, handle.topk_idx, ww, handle.num_tokens, self.group,
                                   out_dtype=x.dtype if x.dtype != torch.float8_e4m3fn else torch.bfloat16)
        return out, w, EventOverlap()

    # ---- low-latency mode ------------------------------------------------------------------------------------
    @_trace.traced("umdk.buffer.low_latency_dispatch")
    def low_latency_dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, num_max_dispatch_tokens_per_rank: int,
                             num_experts: int, use_fp8: bool = True, async_finish: bool = False,
                             return_recv_hook: bool = False, ffn_hidden: Optional[int] = None):
        """-> (recv_x = (slab_fp8 [n_cap, H], scales), recv_count [E_local] int64, handle, event, hook).
        Rows of local expert e occupy slab rows [group_off[e], group_off[e+1]) (`handle.group_off`)."""
        assert x.is_cuda and use_fp8, "the low-latency path is fp8 on CUDA tensors"
        K = topk_idx.shape[1]
        F = ffn_hidden or self._geom_hint[3] or 2048
        st = self._ll_state(num_experts, K, x.shape[1], F, num_max_dispatch_tokens_per_rank)
        st.dispatch(x.contiguous(), topk_idx.contiguous())
        sx, ss, sm = st.slab_views()
        ev = EventOverlap(torch.cuda.current_stream().record_event()) if async_finish else EventOverlap()
        return (sx, ss), st.recv_per_expert, st, ev, (lambda: None) if return_recv_hook else None

    @_trace.traced("umdk.buffer.fused_moe")
    def fused_moe(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, experts, shared=None,
                  num_experts: Optional[int] = None, num_max_tokens_per_rank: Optional[int] = None):
        """dispatch -> expert SwiGLU FFN (fp8, tcgen05) -> combine in one call chain.
        -> (combine_x, share_output, expert_token_nums) like the reference's fused_deep_moe."""
        E = num_experts or self._geom_hint[0] or experts.w1q.shape[0] * self.group_size
        K = topk_idx.shape[1]
        F = experts.w2q.shape[2]
        cap = num_max_tokens_per_rank or max(x.shape[0], 1)
        st = self._ll_state(E, K, x.shape[1], F, cap)
        return st.moe(x.contiguous(), topk_idx.contiguous(), topk_weights.contiguous(), experts, shared)

    @_trace.traced("umdk.buffer.low_latency_combine")
    def low_latency_combine(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, handle,
                            async_finish: bool = False, return_recv_hook: bool = False,
                            out: Optional[torch.Tensor] = None):
        """x: expert outputs [>= N, H] bf16 in the slab row order of `low_latency_dispatch`.
        -> (combined_x [T, H], event, hook). One kernel of its own (ep_ll_combine): rows go back to the token owners
        over NVLink, completion flags, weighted sum; nothing is read back on the host."""
        st = handle
        res = st.combine(x.contiguous(), topk_idx.contiguous(), topk_weights.float().contiguous(), out=out)
        ev = EventOverlap(torch.cuda.current_stream().record_event()) if async_finish else EventOverlap()
        return res, ev, (lambda: None) if return_recv_hook else None
