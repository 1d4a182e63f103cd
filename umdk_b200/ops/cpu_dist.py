"""Expert-parallel dispatch / combine on CPU tensors over a gloo process group.

Used when there is no GPU: it is the transport-level twin of the CUDA kernels (same outputs, same orderings) with
`torch.distributed.all_to_all_single` carrying the counts, the token rows and the per-row metadata. The reference has
no CPU path at all (its tests need 16 Ascend dies, test/cam/ut/test_moe_dispatch_combine_prefill.py:103-167); this
one exists so that the operator contract can be checked anywhere.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from . import reference as ref


@dataclass
class CpuDispatchResult:
    recv_x: torch.Tensor
    recv_scales: Optional[torch.Tensor]
    expand_idx: torch.Tensor            # [N, 3] (srcRank, srcToken, k)
    recv_count: torch.Tensor            # [E_local * R] inclusive prefix (index = le * R + src)
    recv_tokens_per_expert: torch.Tensor  # [E_local] int64
    recv_weights: torch.Tensor          # [N]
    layout: ref.Layout
    num_tokens: int
    quant: bool



def _world(group) -> int:
    """World size of the group; 1 when torch.distributed is not initialised (single-process use)."""
    return dist.get_world_size(group) if dist.is_initialized() else 1


def _all_to_all_single(out, send, output_split_sizes=None, input_split_sizes=None, group=None):
    if not dist.is_initialized():
        out.copy_(send)   # one rank: everything it sends comes back to it
        return
    dist.all_to_all_single(out, send, output_split_sizes=output_split_sizes, input_split_sizes=input_split_sizes,
                           group=group)


def _a2a(send: torch.Tensor, send_splits, recv_splits, group) -> torch.Tensor:
    """Variable-split all-to-all of rows. Rows travel as raw bytes, so any dtype works on gloo."""
    send = send.contiguous()
    tail = tuple(send.shape[1:])
    raw = send.reshape(send.shape[0], -1).view(torch.uint8) if send.shape[0] else \
        torch.empty(0, max(1, send[0:0].reshape(0, -1).shape[1]) * send.element_size(), dtype=torch.uint8)
    row_bytes = raw.shape[1]
    out = torch.empty(sum(recv_splits), row_bytes, dtype=torch.uint8)
    _all_to_all_single(out, raw.contiguous(), output_split_sizes=list(recv_splits),
                       input_split_sizes=list(send_splits), group=group)
    return out.view(send.dtype).reshape((sum(recv_splits),) + tail)


def cpu_dispatch(x: torch.Tensor, topk_idx: torch.Tensor, topk_w: Optional[torch.Tensor], num_experts: int,
                 group=None, quant: bool = False) -> CpuDispatchResult:
    R = _world(group)
    E = num_experts
    el = E // R
    T, K = topk_idx.shape
    H = x.shape[1]
    lay = ref.ref_layout(topk_idx, E, R)
    idx = topk_idx.to(torch.int64)
    w = topk_w.float() if topk_w is not None else torch.ones(T, K)
    # 1. counts: cnt_from[src][le]
    my_counts = lay.num_tokens_per_expert.reshape(R, el).to(torch.int64)
    cnt_from = torch.empty(R, el, dtype=torch.int64)
    _all_to_all_single(cnt_from, my_counts.contiguous(), group=group)
    # 2. rows sorted by (destination expert, bucket position) == (destination rank, local expert, position)
    valid = (idx >= 0) & (idx < E)
    tt, kk = torch.nonzero(valid, as_tuple=True)
    ee = idx[tt, kk]
    pos = lay.send_token_idx[tt, kk].to(torch.int64)
    order = torch.argsort(ee * (T * K + 1) + pos)
    tt, kk, ee = tt[order], kk[order], ee[order]
    send_splits = my_counts.sum(dim=1).tolist()
    recv_splits = cnt_from.sum(dim=1).tolist()
    if quant:
        q, s = ref.quant_fp8_1x128(x)
        rows = _a2a(q[tt].view(torch.uint8), send_splits, recv_splits, group).view(torch.float8_e4m3fn)
        scales = _a2a(s[tt], send_splits, recv_splits, group)
    else:
        payload = x[tt]
        if payload.dtype == torch.bfloat16:  # gloo moves bf16 as raw 16-bit words
            rows = _a2a(payload.view(torch.int16), send_splits, recv_splits, group).view(torch.bfloat16)
        else:
            rows = _a2a(payload, send_splits, recv_splits, group)
        scales = None
    meta = _a2a(torch.stack((tt, kk), dim=1), send_splits, recv_splits, group)
    wts = _a2a(w[tt, kk].unsqueeze(1).contiguous(), send_splits, recv_splits, group).squeeze(1)
    # 3. place: received blocks are (src-major, then local expert); wanted order is (local expert, then src)
    flat = cnt_from.t().reshape(-1)                      # [le * R + src]
    incl = torch.cumsum(flat, dim=0)
    excl = incl - flat
    N = int(incl[-1]) if flat.numel() else 0
    dest = torch.empty(N, dtype=torch.int64)
    src_of = torch.empty(N, dtype=torch.int32)
    cursor = 0
    for s in range(R):
        for le in range(el):
            c = int(cnt_from[s, le])
            if c:
                dest[cursor:cursor + c] = excl[le * R + s] + torch.arange(c)
                src_of[cursor:cursor + c] = s
                cursor += c
    inv = torch.empty(N, dtype=torch.int64)
    inv[dest] = torch.arange(N)
    expand = torch.stack((src_of[inv], meta[inv, 0].to(torch.int32), meta[inv, 1].to(torch.int32)), dim=1) \
        if N else torch.zeros(0, 3, dtype=torch.int32)
    return CpuDispatchResult(rows[inv], scales[inv] if scales is not None else None, expand.to(torch.int32),
                             incl.to(torch.int32), cnt_from.sum(dim=0), wts[inv], lay, T, quant)


def cpu_notify(num_tokens_per_expert: torch.Tensor, num_tokens_per_rank: torch.Tensor, group=None):
    """Count exchange alone on CPU ranks: returns (recv_count inclusive prefix [le*R+src], recv_offset,
    recv_tokens_per_expert, totals[rows, tokens, max tokens from one source]) - the same numbers the GPU operator
    gives (notify_dispatch.h:91-160 in the reference)."""
    R = _world(group)
    el = num_tokens_per_expert.numel() // R
    mine = torch.cat((num_tokens_per_expert.reshape(R, el).to(torch.int64),
                      num_tokens_per_rank.reshape(R, 1).to(torch.int64)), dim=1).contiguous()
    got = torch.empty_like(mine)
    _all_to_all_single(got, mine, group=group)
    flat = got[:, :el].t().reshape(-1)
    incl = torch.cumsum(flat, dim=0)
    arrivals = got[:, el]
    totals = torch.tensor([int(flat.sum()), int(arrivals.sum()), int(arrivals.max()) if R else 0, 0],
                          dtype=torch.int32)
    return incl.to(torch.int32), (incl - flat).to(torch.int32), got[:, :el].sum(dim=0), totals


def cpu_combine(y: torch.Tensor, expand_idx: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor,
                num_tokens: int, group=None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """Returns each row to (srcRank, srcToken, k) and forms sum_k w[t,k] * row in fp32, rounded once."""
    R = _world(group)
    H = y.shape[1]
    src = expand_idx[:, 0].to(torch.int64)
    order = torch.argsort(src, stable=True)
    send_splits = torch.bincount(src, minlength=R).tolist()
    recv_cnt = torch.empty(R, dtype=torch.int64)
    _all_to_all_single(recv_cnt, torch.tensor(send_splits, dtype=torch.int64), group=group)
    recv_splits = recv_cnt.tolist()
    rows = _a2a(y.float()[order], send_splits, recv_splits, group)
    meta = _a2a(expand_idx[order][:, 1:].to(torch.int64).contiguous(), send_splits, recv_splits, group)
    acc = torch.zeros(num_tokens, H, dtype=torch.float32)
    if rows.shape[0]:
        t, k = meta[:, 0], meta[:, 1]
        acc.index_add_(0, t, rows * topk_w.float()[t, k].unsqueeze(1))
    return acc.to(out_dtype)
