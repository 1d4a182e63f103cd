"""Plain-PyTorch statement of the expert-parallel MoE operators. It is the oracle for every CUDA kernel of the
package and the implementation used on CPU (gloo) process groups.

Semantics follow the reference project's operator contract:
  * ``get_dispatch_layout``: src/cam/comm_operator/ascend_kernels/dispatch_layout/op_kernel/dispatch_layout.h:112-165
    (bucket position of (token, k) inside its expert, tokens ascending, then k)
  * receive order "local expert major, then source rank": notify_dispatch/op_kernel/notify_dispatch.h:264-412
  * ``expand_idx`` triples (srcRank, srcToken, k): moe_dispatch_normal/op_kernel/moe_dispatch_normal.h:335-344
  * combine = sum_k w[t,k] * row(t,k) accumulated in fp32, rounded once: moe_combine_normal.h:351-377
The payload format differs on purpose: fp8 e4m3 with one fp32 scale per 1x128 block instead of per-token int8.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

FP8_MAX = 448.0
QBLOCK = 128


# ------------------------------------------------------------------------------------------------------------------
# quantisation helpers
# ------------------------------------------------------------------------------------------------------------------
def quant_fp8_1x128(x: torch.Tensor):
    """x[..., H] -> (q float8_e4m3fn [..., H], scales fp32 [..., H/128]); scale = clamp(amax, 1e-4) / 448."""
    H = x.shape[-1]
    assert H % QBLOCK == 0
    xf = x.float().reshape(*x.shape[:-1], H // QBLOCK, QBLOCK)
    amax = xf.abs().amax(dim=-1).clamp_min(1e-4)
    inv = FP8_MAX / amax
    q = (xf * inv.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(x.shape), (amax * (1.0 / FP8_MAX)).contiguous()


def dequant_fp8_1x128(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    H = q.shape[-1]
    qf = q.float().reshape(*q.shape[:-1], H // QBLOCK, QBLOCK)
    return (qf * scales.unsqueeze(-1)).reshape(q.shape)


def quant_fp8_128x128(w: torch.Tensor):
    """w[..., N, K] -> (q float8_e4m3fn, scales fp32 [..., N/128, K/128])."""
    N, K = w.shape[-2:]
    assert N % QBLOCK == 0 and K % QBLOCK == 0
    wf = w.float().reshape(*w.shape[:-2], N // QBLOCK, QBLOCK, K // QBLOCK, QBLOCK)
    amax = wf.abs().amax(dim=(-3, -1)).clamp_min(1e-4)  # [..., N/128, K/128]
    inv = (FP8_MAX / amax)[..., :, None, :, None]
    q = (wf * inv).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(w.shape), (amax * (1.0 / FP8_MAX)).contiguous()


def dequant_fp8_128x128(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    N, K = q.shape[-2:]
    qf = q.float().reshape(*q.shape[:-2], N // QBLOCK, QBLOCK, K // QBLOCK, QBLOCK)
    return (qf * scales[..., :, None, :, None]).reshape(q.shape)


# ------------------------------------------------------------------------------------------------------------------
# layout
# ------------------------------------------------------------------------------------------------------------------
@dataclass
class Layout:
    num_tokens_per_expert: torch.Tensor  # [E] int32
    num_tokens_per_rank: torch.Tensor    # [R] int32
    is_token_in_rank: torch.Tensor       # [T, R] bool
    send_token_idx: torch.Tensor         # [T, K] int32, position of (t,k) inside expert bucket; -1 for skipped
    rank_slot: torch.Tensor              # [T, R] int32, position of token among those sent to rank r; -1 if absent


def ref_layout(topk_idx: torch.Tensor, num_experts: int, num_ranks: int) -> Layout:
    T, K = topk_idx.shape
    E, R = num_experts, num_ranks
    idx = topk_idx.to(torch.int64)
    valid = (idx >= 0) & (idx < E)
    flat = idx.reshape(-1)
    vflat = valid.reshape(-1)
    onehot = torch.zeros(T * K, E, dtype=torch.int32)
    rows = torch.nonzero(vflat).squeeze(-1)
    onehot[rows, flat[rows]] = 1
    excl = torch.cumsum(onehot, dim=0) - onehot  # entries before (t,k) in (t asc, k asc) order
    send = torch.full((T * K,), -1, dtype=torch.int32)
    send[rows] = excl[rows, flat[rows]].to(torch.int32)
    num_per_expert = onehot.sum(dim=0).to(torch.int32)
    e_local = E // R
    in_rank = torch.zeros(T, R, dtype=torch.bool)
    tt = torch.arange(T).unsqueeze(1).expand(T, K)[valid]
    in_rank[tt, (idx[valid] // e_local)] = True
    ir = in_rank.to(torch.int32)
    rslot = torch.cumsum(ir, dim=0) - ir
    rslot = torch.where(in_rank, rslot, torch.full_like(rslot, -1)).to(torch.int32)
    return Layout(num_per_expert, ir.sum(dim=0).to(torch.int32), in_rank, send.reshape(T, K), rslot)


# ------------------------------------------------------------------------------------------------------------------
# single-process simulation of R ranks (the oracle)
# ------------------------------------------------------------------------------------------------------------------
@dataclass
class DispatchOut:
    recv_x: torch.Tensor            # [N, H] (bf16 or float8_e4m3fn)
    recv_scales: Optional[torch.Tensor]  # [N, H/128] fp32 when quantised
    expand_idx: torch.Tensor        # [N, 3] int32 (srcRank, srcToken, k)
    recv_count: torch.Tensor        # [E_local * R] int32 inclusive prefix, index = le * R + src
    recv_tokens_per_expert: torch.Tensor  # [E_local] int64
    recv_weights: torch.Tensor      # [N] fp32: weight of (srcToken, k)
    # arrival view (one entry per (source token, this rank))
    arr_src: torch.Tensor           # [A] int32
    arr_tok: torch.Tensor           # [A] int32
    arr_rows: torch.Tensor          # [A, K] int32, row per k or -1
    arr_w: torch.Tensor             # [A, K] fp32


def ref_dispatch_all(xs: Sequence[torch.Tensor], topk_idxs: Sequence[torch.Tensor],
                     topk_ws: Sequence[Optional[torch.Tensor]], num_experts: int, quant: bool) -> List[DispatchOut]:
    """Dispatch for all R ranks at once. xs[r]: [T_r, H] bf16/fp32; returns one DispatchOut per rank."""
    R = len(xs)
    E = num_experts
    e_local = E // R
    K = topk_idxs[0].shape[1]
    H = xs[0].shape[1]
    layouts = [ref_layout(t.cpu(), E, R) for t in topk_idxs]
    outs = []
    for d in range(R):
        # counts[le][src]
        cnt = torch.zeros(e_local, R, dtype=torch.int64)
        for s in range(R):
            cnt[:, s] = layouts[s].num_tokens_per_expert[d * e_local:(d + 1) * e_local].to(torch.int64)
        flat = cnt.reshape(-1)
        incl = torch.cumsum(flat, dim=0)
        excl = incl - flat
        N = int(incl[-1].item()) if flat.numel() else 0
        dt = torch.float8_e4m3fn if quant else xs[0].dtype
        recv_x = torch.zeros(N, H, dtype=dt)
        recv_s = torch.zeros(N, H // QBLOCK, dtype=torch.float32) if quant else None
        expand = torch.zeros(N, 3, dtype=torch.int32)
        recv_w = torch.zeros(N, dtype=torch.float32)
        arr_src, arr_tok, arr_rows, arr_w = [], [], [], []
        for s in range(R):
            idx = topk_idxs[s].cpu().to(torch.int64)
            lay = layouts[s]
            toks = torch.nonzero(lay.is_token_in_rank[:, d]).squeeze(-1)
            if toks.numel() == 0:
                continue
            xsrc = xs[s].cpu()[toks]
            if quant:
                q, sc = quant_fp8_1x128(xsrc)
            w_all = topk_ws[s].cpu().float() if topk_ws[s] is not None else torch.ones(idx.shape, dtype=torch.float32)
            rows = torch.full((toks.numel(), K), -1, dtype=torch.int32)
            for k in range(K):
                e = idx[toks, k]
                mine = (e >= 0) & (e < E) & ((e // e_local) == d)
                le = (e % e_local)
                r = excl[(le * R + s).clamp(0, flat.numel() - 1)] + lay.send_token_idx[toks, k].to(torch.int64)
                sel = torch.nonzero(mine).squeeze(-1)
                rr = r[sel]
                rows[sel, k] = rr.to(torch.int32)
                if quant:
                    recv_x[rr] = q[sel]
                    recv_s[rr] = sc[sel]
                else:
                    recv_x[rr] = xsrc[sel].to(dt)
                expand[rr, 0] = s
                expand[rr, 1] = toks[sel].to(torch.int32)
                expand[rr, 2] = k
                recv_w[rr] = w_all[toks[sel], k]
            arr_src.append(torch.full((toks.numel(),), s, dtype=torch.int32))
            arr_tok.append(toks.to(torch.int32))
            arr_rows.append(rows)
            arr_w.append(w_all[toks])
        cat = lambda lst, shape, dtp: torch.cat(lst) if lst else torch.zeros(shape, dtype=dtp)
        outs.append(DispatchOut(
            recv_x, recv_s, expand, incl.to(torch.int32), cnt.sum(dim=1),
            recv_w, cat(arr_src, (0,), torch.int32), cat(arr_tok, (0,), torch.int32),
            cat(arr_rows, (0, K), torch.int32), cat(arr_w, (0, K), torch.float32)))
    return outs


def ref_combine_all(ys: Sequence[torch.Tensor], disp: Sequence[DispatchOut], topk_idxs: Sequence[torch.Tensor],
                    topk_ws: Sequence[torch.Tensor], out_dtype=torch.bfloat16) -> List[torch.Tensor]:
    """out_r[t] = round( sum_k w_r[t,k] * float(y_row(t,k)) ); ys[d]: [N_d, H] expert outputs on rank d."""
    R = len(ys)
    H = ys[0].shape[1]
    outs = []
    for r in range(R):
        T, K = topk_idxs[r].shape
        acc = torch.zeros(T, H, dtype=torch.float32)
        w = topk_ws[r].cpu().float()
        for d in range(R):
            ex = disp[d].expand_idx
            sel = torch.nonzero(ex[:, 0] == r).squeeze(-1)
            if sel.numel() == 0:
                continue
            t = ex[sel, 1].to(torch.int64)
            k = ex[sel, 2].to(torch.int64)
            acc.index_add_(0, t, ys[d].cpu().float()[sel] * w[t, k].unsqueeze(1))
        outs.append(acc.to(out_dtype))
    return outs


def dense_moe_reference(x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, expert_fn) -> torch.Tensor:
    """out[t] = sum_k w[t,k] * expert_fn(e=topk_idx[t,k], x[t]) computed densely in fp32 (no communication)."""
    T, K = topk_idx.shape
    out = torch.zeros(x.shape, dtype=torch.float32)
    for k in range(K):
        e = topk_idx[:, k]
        for ee in torch.unique(e).tolist():
            if ee < 0:
                continue
            sel = torch.nonzero(e == ee).squeeze(-1)
            out[sel] += topk_w[sel, k].float().unsqueeze(1) * expert_fn(int(ee), x[sel].float())
    return out


def calc_diff(a: torch.Tensor, b: torch.Tensor) -> float:
    """1 - cosine-like similarity used by the reference's samples (src/cam/examples/utils.py `calc_diff`)."""
    a = a.double() + 1
    b = b.double() + 1
    sim = 2 * (a * b).sum() / ((a * a).sum() + (b * b).sum())
    return float(1 - sim)


def mean_rel_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    """Mean relative error, the accuracy metric of the reference's API guide (<= 0.5 % / <= 1 % with quant)."""
    a = a.double()
    ref = ref.double()
    return float(((a - ref).abs().sum() / ref.abs().sum().clamp_min(1e-12)))


def max_row_rel_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    """Largest per-row relative error sum|a - ref| / sum|ref|: one wrong or missing row shows up here even when the
    mean over the whole tensor hides it."""
    a = a.double()
    ref = ref.double()
    num = (a - ref).abs().sum(dim=-1)
    den = ref.abs().sum(dim=-1).clamp_min(1e-12)
    return float((num / den).max())


# ------------------------------------------------------------------------------------------------------------------
# expert FFN (fp8 block-scaled) reference
# ------------------------------------------------------------------------------------------------------------------
def ref_gemm1_swiglu_quant(xq, xs, group_off, w1q, w1s):
    """fp32 statement of the gate/up projection + SwiGLU + fp8 1x128 re-quantisation, group by group.
    Returns (hq float8 [N, F], hs fp32 [N, F/128], h fp32 [N, F] before quantisation)."""
    N = xq.shape[0]
    F = w1q.shape[1] // 2
    x = dequant_fp8_1x128(xq.cpu(), xs.cpu())
    h = torch.zeros(N, F, dtype=torch.float32)
    off = group_off.cpu().tolist()
    for g in range(w1q.shape[0]):
        a, b = off[g], off[g + 1]
        if b <= a:
            continue
        w = dequant_fp8_128x128(w1q[g].cpu(), w1s[g].cpu())
        y1 = x[a:b] @ w.t()
        gate, up = y1[:, :F], y1[:, F:]
        h[a:b] = torch.nn.functional.silu(gate) * up
    hq, hs = quant_fp8_1x128(h)
    return hq, hs, h


def ref_gemm2(hq, hs, group_off, w2q, w2s):
    N = hq.shape[0]
    H = w2q.shape[1]
    hdeq = dequant_fp8_1x128(hq.cpu(), hs.cpu())
    y = torch.zeros(N, H, dtype=torch.float32)
    off = group_off.cpu().tolist()
    for g in range(w2q.shape[0]):
        a, b = off[g], off[g + 1]
        if b <= a:
            continue
        w = dequant_fp8_128x128(w2q[g].cpu(), w2s[g].cpu())
        y[a:b] = hdeq[a:b] @ w.t()
    return y


def ref_fused_moe(x, topk_idx, topk_w, w1q, w1s, w2q, w2s):
    """Dense fp32 statement of the low-latency MoE layer for ONE rank's tokens against ALL experts:
    x -> fp8 1x128 -> W1 (fp8 128x128) -> SwiGLU -> fp8 1x128 -> W2 -> bf16 rows -> sum_k w[t,k] * row (fp32).
    w1q: [E, 2F, H], w2q: [E, H, F] over the global expert index."""
    T, K = topk_idx.shape
    xq, xs = quant_fp8_1x128(x.cpu())
    xd = dequant_fp8_1x128(xq, xs)
    F = w1q.shape[1] // 2
    out = torch.zeros(T, w2q.shape[1], dtype=torch.float32)
    idx = topk_idx.cpu()
    w = topk_w.cpu().float()
    for e in torch.unique(idx).tolist():
        if e < 0:
            continue
        tk = torch.nonzero(idx == e)
        t, k = tk[:, 0], tk[:, 1]
        w1 = dequant_fp8_128x128(w1q[e].cpu(), w1s[e].cpu())
        w2 = dequant_fp8_128x128(w2q[e].cpu(), w2s[e].cpu())
        y1 = xd[t] @ w1.t()
        h = torch.nn.functional.silu(y1[:, :F]) * y1[:, F:]
        hq, hs = quant_fp8_1x128(h)
        y2 = (dequant_fp8_1x128(hq, hs) @ w2.t()).to(torch.bfloat16).float()
        out.index_add_(0, t, y2 * w[t, k].unsqueeze(1))
    return out


def ref_moe_unquantised(x, topk_idx, topk_w, w1q, w1s, w2q, w2s):
    """The same layer computed in fp32 from the bf16 activations WITHOUT quantising them (the fp8 weights are what
    the model stores, so they are used as given): the yardstick of the reference's accuracy requirement
    (doc/en/cam/CAM API Guide.md:146-148: mean relative error of combine_x against an unquantised computation)."""
    T, K = topk_idx.shape
    xf = x.float().cpu()
    F = w1q.shape[1] // 2
    out = torch.zeros(T, w2q.shape[1], dtype=torch.float32)
    idx = topk_idx.cpu()
    w = topk_w.cpu().float()
    for e in torch.unique(idx).tolist():
        if e < 0:
            continue
        tk = torch.nonzero(idx == e)
        t, k = tk[:, 0], tk[:, 1]
        w1 = dequant_fp8_128x128(w1q[e].cpu(), w1s[e].cpu())
        w2 = dequant_fp8_128x128(w2q[e].cpu(), w2s[e].cpu())
        y1 = xf[t] @ w1.t()
        h = torch.nn.functional.silu(y1[:, :F]) * y1[:, F:]
        out.index_add_(0, t, (h @ w2.t()) * w[t, k].unsqueeze(1))
    return out

