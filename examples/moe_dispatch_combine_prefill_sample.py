#!/usr/bin/env python
"""Normal-mode (prefill) expert parallelism end to end: get_dispatch_layout -> dispatch -> identity experts ->
combine, checked against the dense statement of the same computation, then timed.

    python examples/moe_dispatch_combine_prefill_sample.py                       # one GPU (or CPU without one)
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        examples/moe_dispatch_combine_prefill_sample.py --tokens 4096

Same flow and defaults as the reference sample (src/cam/examples/moe_dispatch_combine_prefill_sample.py:213-267:
1024 tokens, hidden 7168, top-8, warm-up + timed iterations, GB/s and microseconds per op), on the
DeepEP-style Buffer of this package.
"""
from __future__ import annotations

import argparse
import json

import torch

from utils import bench, init_dist, routing


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--experts-per-rank", type=int, default=32)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--no-fp8", action="store_true")
    a = ap.parse_args()
    rank, world, group = init_dist()
    from umdk_b200 import Buffer
    from umdk_b200.ops import reference as ref
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda") if cuda else torch.device("cpu")
    E = a.experts_per_rank * world
    K = min(a.topk, E)
    g = torch.Generator().manual_seed(rank)
    x = torch.randn(a.tokens, a.hidden, generator=g).to(torch.bfloat16).to(dev)
    idx, w = routing(a.tokens, E, K, 100 + rank, dev)
    buf = Buffer(group, num_experts=E, hidden=a.hidden, top_k=K, max_tokens_per_rank=a.tokens)

    n_rank, _, n_exp, in_rank, _ = buf.get_dispatch_layout(idx, E)
    recv_x, recv_expert, recv_w, per_expert, handle, _ = buf.dispatch(
        x, topk_idx=idx, topk_weights=w, num_tokens_per_rank=n_rank, is_token_in_rank=in_rank,
        num_tokens_per_expert=n_exp, use_fp8=not a.no_fp8)
    if a.no_fp8:
        y = recv_x
    else:
        y = ref.dequant_fp8_1x128(recv_x[0], recv_x[1]).to(torch.bfloat16)
    out, _, _ = buf.combine(y, handle)
    # identity experts: combine(dispatch(x)) == x * sum_k w[t, k] over the selected experts (all of them here)
    want = x.float() * w.sum(-1, keepdim=True).to(x.device)
    err = ref.mean_rel_err(out.float().cpu(), want.cpu())
    tol = 5e-3 if a.no_fp8 else 3e-2
    ok = err < tol
    if rank == 0:
        print(json.dumps({"check": "combine(dispatch(x))", "mean_rel_err": err, "tolerance": tol, "ok": bool(ok),
                          "recv_tokens_rank0": int(sum(per_expert))}))
    assert ok, err
    if cuda:
        row_bytes = a.hidden + (a.hidden // 128) * 4 if not a.no_fp8 else a.hidden * 2
        n_recv = int(sum(per_expert))
        t_d = bench(lambda: buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_expert=n_exp,
                                         use_fp8=not a.no_fp8), a.warmup, a.iters)
        t_c = bench(lambda: buf.combine(y, handle), a.warmup, a.iters)
        if rank == 0:
            print(json.dumps({"op": "dispatch", "avg_us": t_d[0] * 1e6, "min_us": t_d[1] * 1e6,
                              "recv_GBps": n_recv * row_bytes / t_d[0] / 1e9}))
            print(json.dumps({"op": "combine", "avg_us": t_c[0] * 1e6, "min_us": t_c[1] * 1e6,
                              "recv_GBps": a.tokens * K * a.hidden * 2 / t_c[0] / 1e9}))
    buf.destroy()


if __name__ == "__main__":
    main()
