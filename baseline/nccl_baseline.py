"""Plain PyTorch + NCCL (+cuBLAS) statements of the benchmarked pipelines, used as the comparison baseline.

The reference project has no CUDA path to run on this hardware, so the baseline reproduces its *algorithm split* with
library collectives: layout on the GPU -> all_to_all_single of the counts -> separate quantisation kernel ->
all_to_all_single of tokens and scales -> expert compute -> all_to_all_single back -> weighted index_add.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def quant_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    T, H = x.shape
    xf = x.float().view(T, H // 128, 128)
    amax = xf.abs().amax(dim=-1).clamp_min(1e-4)
    q = (xf * (448.0 / amax).unsqueeze(-1)).to(torch.float8_e4m3fn).view(T, H)
    return q, amax / 448.0


def dequant_1x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    T, H = q.shape
    return (q.float().view(T, H // 128, 128) * s.unsqueeze(-1)).view(T, H)


class NcclEp:
    """Dispatch / combine with NCCL all_to_all_single. One row per (token, k), rows sorted by destination expert."""

    def __init__(self, group, num_experts: int):
        self.group = group
        self.R = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E = num_experts
        self.el = num_experts // self.R

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, quant: bool):
        T, K = topk_idx.shape
        flat = topk_idx.reshape(-1)
        order = torch.argsort(flat, stable=True)          # rows by expert, stable in (t, k)
        tok = order // K
        counts = torch.bincount(flat, minlength=self.E)
        send_counts = counts.view(self.R, self.el)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        in_splits = send_counts.sum(1).tolist()           # host sync, as in the reference's .item() calls
        out_splits = recv_counts.sum(1).tolist()
        rows = x[tok]
        if quant:
            q, s = quant_1x128(rows)
            recv_q = torch.empty(sum(out_splits), x.shape[1], dtype=torch.uint8, device=x.device)
            dist.all_to_all_single(recv_q, q.view(torch.uint8), out_splits, in_splits, group=self.group)
            recv_s = torch.empty(sum(out_splits), s.shape[1], dtype=torch.float32, device=x.device)
            dist.all_to_all_single(recv_s, s, out_splits, in_splits, group=self.group)
            recv = (recv_q.view(torch.float8_e4m3fn), recv_s)
        else:
            r = torch.empty(sum(out_splits), x.shape[1], dtype=x.dtype, device=x.device)
            dist.all_to_all_single(r, rows, out_splits, in_splits, group=self.group)
            recv = r
        return recv, dict(order=order, in_splits=in_splits, out_splits=out_splits, recv_counts=recv_counts, T=T, K=K)

    def combine(self, y: torch.Tensor, h: dict, topk_w: torch.Tensor) -> torch.Tensor:
        back = torch.empty(sum(h["in_splits"]), y.shape[1], dtype=y.dtype, device=y.device)
        dist.all_to_all_single(back, y, h["in_splits"], h["out_splits"], group=self.group)
        order = h["order"]
        tok, k = order // h["K"], order % h["K"]
        out = torch.zeros(h["T"], y.shape[1], dtype=torch.float32, device=y.device)
        out.index_add_(0, tok, back.float() * topk_w[tok, k].unsqueeze(1))
        return out.to(torch.bfloat16)


def expert_ffn_bf16(recv_q, recv_s, recv_counts, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """Per-expert SwiGLU FFN with cuBLAS bf16 GEMMs on dequantised inputs. Rows arrive grouped by source rank, then
    by local expert; w1 [el, 2F, H], w2 [el, H, F] are bf16 copies of the fp8 weights."""
    x = dequant_1x128(recv_q, recv_s).to(torch.bfloat16)
    R, el = recv_counts.shape
    cnt = recv_counts.tolist()
    y = torch.empty(x.shape[0], w2.shape[1], dtype=torch.bfloat16, device=x.device)
    F = w1.shape[1] // 2
    pos = 0
    for s in range(R):
        for e in range(el):
            c = cnt[s][e]
            if c:
                h1 = x[pos:pos + c] @ w1[e].t()
                hh = torch.nn.functional.silu(h1[:, :F]) * h1[:, F:]
                y[pos:pos + c] = hh @ w2[e].t()
                pos += c
    return y
