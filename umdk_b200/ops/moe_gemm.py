"""Grouped fp8 block-scaled expert GEMMs (csrc/cam/moe_gemm.cu): gate/up projection fused with SwiGLU and fp8
re-quantisation, and the down projection with a local bf16 output or with the combine fused into its epilogue."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native

MAX_RANKS = 32


class MoeGemmParams(ctypes.Structure):
    _fields_ = [
        ("mode", ctypes.c_int), ("G", ctypes.c_int), ("Nout", ctypes.c_int), ("K", ctypes.c_int),
        ("n_rows_cap", ctypes.c_int), ("max_ctas", ctypes.c_int),
        ("w", ctypes.c_void_p), ("ws", ctypes.c_void_p), ("x", ctypes.c_void_p), ("xs", ctypes.c_void_p),
        ("group_off", ctypes.c_void_p), ("hq", ctypes.c_void_p), ("hs", ctypes.c_void_p), ("y", ctypes.c_void_p),
        ("wait_flags", ctypes.c_void_p * 2), ("wait_n", ctypes.c_int), ("epoch_ptr", ctypes.c_void_p),
        ("R", ctypes.c_int), ("rank", ctypes.c_int), ("T", ctypes.c_int), ("Kt", ctypes.c_int),
        ("T_cap", ctypes.c_int),
        ("peers", ctypes.c_void_p * MAX_RANKS),
        ("comb_buf_off", ctypes.c_uint64 * 2), ("comb_flag_off", ctypes.c_uint64 * 2),
        ("row_meta", ctypes.c_void_p), ("topk_idx", ctypes.c_void_p), ("topk_w", ctypes.c_void_p),
        ("out", ctypes.c_void_p), ("ctrl", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("phase_mask", ctypes.c_int),
    ]


def _base(mode, w, ws, x, xs, group_off, status, max_ctas=0) -> MoeGemmParams:
    assert w.is_cuda and w.is_contiguous() and x.is_contiguous() and ws.is_contiguous() and xs.is_contiguous()
    assert group_off.dtype == torch.int32
    p = MoeGemmParams()
    G, w_rows, K = w.shape
    p.mode, p.G, p.K = mode, G, K
    p.Nout = w_rows // 2 if mode == 0 else w_rows
    p.n_rows_cap, p.max_ctas = x.shape[0], max_ctas
    p.w, p.ws, p.x, p.xs = w.data_ptr(), ws.data_ptr(), x.data_ptr(), xs.data_ptr()
    p.group_off = group_off.data_ptr()
    p.status = status.data_ptr()
    return p


def gemm1_swiglu_quant(xq, xs, group_off, w1q, w1s, status, hq=None, hs=None, wait_flags=None, wait_n=0,
                       epoch_ptr=0, max_ctas=0):
    """h = SwiGLU(x @ W1^T) re-quantised to fp8 1x128. w1q: [G, 2F, K] (gate rows first)."""
    lib = _native.cam()
    p = _base(0, w1q, w1s, xq, xs, group_off, status, max_ctas)
    F = p.Nout
    n = xq.shape[0]
    if hq is None:
        hq = torch.empty(n, F, dtype=torch.uint8, device=xq.device).view(torch.float8_e4m3fn)
        hs = torch.empty(n, F // 128, dtype=torch.float32, device=xq.device)
    p.hq, p.hs = hq.data_ptr(), hs.data_ptr()
    if wait_flags is not None:
        p.wait_flags[0], p.wait_flags[1] = wait_flags
        p.wait_n, p.epoch_ptr = wait_n, epoch_ptr
    rc = lib.umdk_moe_gemm(ctypes.byref(p), _native.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"umdk_moe_gemm(mode 0) failed: {rc}")
    return hq, hs


def gemm2(hq, hs, group_off, w2q, w2s, status, y=None, max_ctas=0):
    """y = h @ W2^T as bf16 rows in local memory. w2q: [G, H, F]."""
    lib = _native.cam()
    p = _base(1, w2q, w2s, hq, hs, group_off, status, max_ctas)
    if y is None:
        y = torch.empty(hq.shape[0], p.Nout, dtype=torch.bfloat16, device=hq.device)
    p.y = y.data_ptr()
    rc = lib.umdk_moe_gemm(ctypes.byref(p), _native.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"umdk_moe_gemm(mode 1) failed: {rc}")
    return y
