"""Sparse top-k MLA flash-attention decode over a paged KV cache (csrc/cam/sparse_mla_decode.cu): one cluster of two
CTAs per (sequence, key-list split), the feature dimensions divided between them."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native

HEADS = 128
DIM = 576
DIM_V = 512
PAGE = 64


def sparse_mla_decode(q: torch.Tensor, kv_pages: torch.Tensor, block_table: torch.Tensor, indices: torch.Tensor,
                      sm_scale: float, seq_lens: Optional[torch.Tensor] = None, num_splits: int = 0,
                      out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                      workspace: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                      diag: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [B,128,576] bf16, kv_pages [P,64,576] bf16, block_table [B,max_pages] int32, indices [B,topk] int32
    (token positions; -1 = unused) -> (out [B,128,512] bf16, lse [B,128] fp32).
    ``num_splits`` 0 = as many splits of the key list as it takes to put a CTA pair on every SM (a batch of 64
    already does with one split), each split keeping at least four 48-key chunks.
    ``diag`` (int64 [16], device): the first CTA records how many cycles its roles spent in each of their waits and
    work sections (see MlaArgs::diag in the kernel source); for finding what bounds the pipeline."""
    lib = _native.cam()
    assert q.is_cuda and q.dtype == torch.bfloat16 and q.is_contiguous() and q.shape[1:] == (HEADS, DIM)
    assert kv_pages.dtype == torch.bfloat16 and kv_pages.is_contiguous() and kv_pages.shape[1:] == (PAGE, DIM)
    assert block_table.dtype == torch.int32 and indices.dtype == torch.int32
    assert block_table.is_contiguous() and indices.is_contiguous()
    B = q.shape[0]
    topk = indices.shape[1]
    dev = q.device
    if out is None:
        out = torch.empty(B, HEADS, DIM_V, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(B, HEADS, dtype=torch.float32, device=dev)
    if status is None:
        status = torch.zeros(4, dtype=torch.int32, device=dev)
    # one CTA pair resolves at most 2064 selected rows up front: longer key lists need more splits
    if num_splits <= 0:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        num_splits = max(1, min(sms // (2 * B), topk // (4 * 48), 16))
    num_splits = max(num_splits, int(lib.umdk_sparse_mla_min_splits(topk)))
    if workspace is not None and workspace[0].shape[1] != num_splits:
        workspace = None
    po = pl = None
    if num_splits > 1:
        if workspace is None:
            workspace = (torch.empty(B, num_splits, HEADS, DIM_V, dtype=torch.float32, device=dev),
                         torch.empty(B, num_splits, HEADS, dtype=torch.float32, device=dev))
        po, pl = workspace
    import ctypes
    rc = lib.umdk_sparse_mla_decode(
        _native.ptr(q), _native.ptr(kv_pages), _native.ptr(block_table), _native.ptr(indices),
        _native.ptr(seq_lens), _native.ptr(out), _native.ptr(lse), _native.ptr(po), _native.ptr(pl),
        B, topk, block_table.shape[1], kv_pages.shape[0], num_splits, ctypes.c_float(sm_scale),
        _native.ptr(status), _native.stream_ptr(), _native.ptr(diag))
    if rc != 0:
        raise RuntimeError(f"umdk_sparse_mla_decode failed: {rc}")
    return out, lse


def ref_sparse_mla_decode(q, kv_pages, block_table, indices, sm_scale, seq_lens=None):
    """fp32 PyTorch statement of the same op (gather rows, masked softmax, weighted sum of the 512-wide values)."""
    B = q.shape[0]
    qf = q.float().cpu()
    kv = kv_pages.float().cpu().reshape(-1, DIM)
    bt = block_table.cpu().long()
    idx = indices.cpu().long()
    out = torch.zeros(B, HEADS, DIM_V)
    lse = torch.full((B, HEADS), float("-inf"))
    for b in range(B):
        valid = idx[b] >= 0
        if seq_lens is not None:
            valid &= idx[b] < int(seq_lens[b])
        pos = idx[b][valid]
        if pos.numel() == 0:
            continue
        rows = bt[b][pos // PAGE] * PAGE + pos % PAGE
        k = kv[rows]
        s = (qf[b] @ k.t()) * sm_scale
        lse[b] = torch.logsumexp(s, dim=-1)
        out[b] = torch.softmax(s, dim=-1) @ k[:, :DIM_V]
    return out, lse
