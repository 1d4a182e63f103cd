#!/usr/bin/env python
"""Low-latency (decode) MoE layer: the fused path (dispatch -> grouped fp8 GEMM1 + SwiGLU + re-quant -> GEMM2 with the
combine in its epilogue) against a "small ops" pipeline that runs the same layer as separate steps - normal-mode
dispatch, dequantise, per-expert bf16 matmuls, SwiGLU, normal-mode combine - the comparison the reference's sample
makes between its fused operator and `SmallOps` (src/cam/examples/fused_deep_moe_sample.py:125-229, 485).

    python examples/fused_deep_moe_sample.py
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/fused_deep_moe_sample.py
"""
from __future__ import annotations

import argparse
import json

import torch

from utils import bench, init_dist, routing


def small_ops(buf, x, idx, w, experts, E):
    from umdk_b200.ops import reference as ref
    n_rank, _, n_exp, in_rank, _ = buf.get_dispatch_layout(idx, E)
    (rq, rs), _, _, per_expert, handle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_expert=n_exp)
    xin = ref.dequant_fp8_1x128(rq, rs)
    y = torch.empty(xin.shape[0], x.shape[1], dtype=torch.bfloat16, device=x.device)
    r0 = 0
    for e, n in enumerate(per_expert):
        if n == 0:
            continue
        w1 = ref.dequant_fp8_128x128(experts.w1q[e:e + 1], experts.w1s[e:e + 1])[0]
        w2 = ref.dequant_fp8_128x128(experts.w2q[e:e + 1], experts.w2s[e:e + 1])[0]
        h = xin[r0:r0 + n] @ w1.t()
        F = h.shape[1] // 2
        h = torch.nn.functional.silu(h[:, :F]) * h[:, F:]
        y[r0:r0 + n] = (h @ w2.t()).to(torch.bfloat16)
        r0 += n
    out, _, _ = buf.combine(y, handle)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    rank, world, group = init_dist()
    assert torch.cuda.is_available(), "the fused low-latency path needs a GPU"
    from umdk_b200 import Buffer
    from umdk_b200.models.dsv3_decoder import _quant_experts
    from umdk_b200.ops import reference as ref
    from umdk_b200.ops.ep_ll import ExpertWeights
    dev = torch.device("cuda")
    E, K, el = a.experts, a.topk, a.experts // world
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    x = torch.randn(a.tokens, a.hidden, device=dev, generator=g).to(torch.bfloat16)
    idx, w = routing(a.tokens, E, K, 100 + rank, dev)
    experts = ExpertWeights(*_quant_experts(el, 2 * a.ffn, a.hidden, dev, g), *_quant_experts(el, a.hidden, a.ffn, dev, g))
    buf = Buffer(group, low_latency_mode=True, num_experts=E, hidden=a.hidden, top_k=K, ffn_hidden=a.ffn,
                 max_tokens_per_rank=a.tokens)
    fused, _, counts = buf.fused_moe(x, idx, w, experts, num_experts=E, num_max_tokens_per_rank=a.tokens)
    small = small_ops(buf, x, idx, w, experts, E)
    torch.cuda.synchronize()
    err = ref.mean_rel_err(fused.float().cpu(), small.float().cpu())
    if rank == 0:
        print(json.dumps({"check": "fused vs small ops", "mean_rel_err": err, "tolerance": 0.03, "ok": err < 0.03,
                          "tokens_on_rank0_experts": int(counts.sum())}))
    assert err < 0.03, err
    t_f = bench(lambda: buf.fused_moe(x, idx, w, experts, num_experts=E, num_max_tokens_per_rank=a.tokens),
                a.warmup, a.iters)
    t_s = bench(lambda: small_ops(buf, x, idx, w, experts, E), 2, 5)
    if rank == 0:
        print(json.dumps({"fused_us": t_f[0] * 1e6, "small_ops_us": t_s[0] * 1e6, "speedup": t_s[0] / t_f[0]}))
    buf.destroy()


if __name__ == "__main__":
    main()
