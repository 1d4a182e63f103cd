"""Fused small kernels of the decode step (csrc/cam/decoder_glue.cu): residual add + RMSNorm, the post-processing of
the fused q_a / kv_a projection (q RMSNorm; KV RMSNorm + rotary embedding + write of the token's KV row), the rotary
part of the absorbed query, and the router (softmax + top-k + renormalisation + folded expert numbering)."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .. import _native

# what torch.nn.functional.rms_norm uses when eps is None: the epsilon of its fp32 accumulation type
RMS_EPS = float(torch.finfo(torch.float32).eps)


def _chk(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed: {rc}")


def add_rmsnorm(x: torch.Tensor, w: torch.Tensor, a: Optional[torch.Tensor] = None,
                b: Optional[torch.Tensor] = None, x_out: Optional[torch.Tensor] = None,
                h: Optional[torch.Tensor] = None, eps: float = RMS_EPS) -> Tuple[torch.Tensor, torch.Tensor]:
    """(x + a + b, rmsnorm(x + a + b) * w) in one launch; with no addends the first result is ``x`` itself."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    T, H = x.shape
    if h is None:
        h = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    if a is None and b is None:
        x_out = None
    elif x_out is None:
        x_out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    for t in (a, b):
        assert t is None or (t.is_contiguous() and t.shape == (T, H) and t.dtype == torch.bfloat16)
    _chk(_native.cam().umdk_add_rmsnorm(_native.ptr(x), _native.ptr(a), _native.ptr(b), _native.ptr(w),
                                        _native.ptr(x_out), _native.ptr(h), T, H, x.stride(0), ctypes.c_float(eps),
                                        _native.stream_ptr()), "umdk_add_rmsnorm")
    return (x_out if x_out is not None else x), h


def qkv_post(qkv: torch.Tensor, q_lora: int, q_norm: torch.Tensor, kv_norm: torch.Tensor, cos: torch.Tensor,
             sin: torch.Tensor, kv_pool: torch.Tensor, new_row: torch.Tensor, status: torch.Tensor,
             qa: Optional[torch.Tensor] = None, eps: float = RMS_EPS) -> torch.Tensor:
    """qkv [T, q_lora + 576] bf16 -> qa [T, q_lora]; writes row new_row[t] (int64, in rows of 576) of ``kv_pool``."""
    T = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == q_lora + 576 and new_row.dtype == torch.int64
    assert cos.dtype == torch.float32 and cos.numel() == 32 and kv_pool.is_contiguous()
    if qa is None:
        qa = torch.empty(T, q_lora, dtype=torch.bfloat16, device=qkv.device)
    _chk(_native.cam().umdk_qkv_post(_native.ptr(qkv), T, q_lora, _native.ptr(q_norm), _native.ptr(kv_norm),
                                     _native.ptr(cos), _native.ptr(sin), _native.ptr(qa), _native.ptr(kv_pool),
                                     _native.ptr(new_row), ctypes.c_longlong(kv_pool.numel() // 576),
                                     ctypes.c_float(eps), _native.ptr(status), _native.stream_ptr()), "umdk_qkv_post")
    return qa


def q_rope(q: torch.Tensor, nope: int, cos: torch.Tensor, sin: torch.Tensor, q_full: torch.Tensor):
    """q [T, heads, nope + 64] -> q_full[T, heads, 512:576] = rotary(q[..., nope:])."""
    assert q.is_contiguous() and q_full.is_contiguous() and q_full.shape[-1] == 576
    rows = q.shape[0] * q.shape[1]
    _chk(_native.cam().umdk_q_rope(_native.ptr(q), rows, q.shape[2], nope, _native.ptr(cos), _native.ptr(sin),
                                   _native.ptr(q_full), _native.stream_ptr()), "umdk_q_rope")


def router_topk(logits: torch.Tensor, k: int, fold_el: int = 0, rank: int = 0):
    """logits [T, E] bf16 -> (idx [T, k(+1)] int64, w [T, k(+1)] fp32): top-k of the softmax with weights renormalised
    over the winners. ``fold_el`` > 0: ids renumbered for ranks that own fold_el routed experts plus one shared expert,
    and one more slot that selects rank ``rank``'s shared expert with weight 1 (EpLowLatency fold_shared)."""
    assert logits.is_cuda and logits.dtype == torch.bfloat16 and logits.is_contiguous()
    T, E = logits.shape
    ko = k + (1 if fold_el > 0 else 0)
    idx = torch.empty(T, ko, dtype=torch.int64, device=logits.device)
    w = torch.empty(T, ko, dtype=torch.float32, device=logits.device)
    _chk(_native.cam().umdk_router_topk(_native.ptr(logits), T, E, k, fold_el, rank, _native.ptr(idx), _native.ptr(w),
                                        _native.stream_ptr()), "umdk_router_topk")
    return idx, w
