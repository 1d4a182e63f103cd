"""The NCCL(+library GEMM) comparison baseline is itself checked against the dense fp32 oracle, on CPU: one process
and two gloo ranks. A baseline that computes something else would make every speed-up quoted against it meaningless."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from baseline.nccl_baseline import GroupedFfn, NcclEp, NcclLowLatencyMoe
from umdk_b200.ops import reference as ref


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _experts(n, F, H, seed):
    g = torch.Generator().manual_seed(seed)
    w1q, w1s = ref.quant_fp8_128x128(torch.randn(n, 2 * F, H, generator=g) * 0.05)
    w2q, w2s = ref.quant_fp8_128x128(torch.randn(n, H, F, generator=g) * 0.05)
    return w1q, w1s, w2q, w2s


def _inputs(rank, T, H, E, K):
    g = torch.Generator().manual_seed(10 + rank)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    p = torch.softmax(torch.randn(T, E, generator=g), dim=-1)
    w, idx = torch.topk(p, K, dim=-1)
    idx = idx.to(torch.int64)
    idx[::7, K - 1] = -1
    return x, idx, (w / w.sum(-1, keepdim=True)).float()


def _dense(x, idx, w, all_experts, F):
    w1q, w1s, w2q, w2s = all_experts
    def fn(e, rows):
        w1 = ref.dequant_fp8_128x128(w1q[e], w1s[e])
        w2 = ref.dequant_fp8_128x128(w2q[e], w2s[e])
        h1 = rows @ w1.t()
        return (torch.nn.functional.silu(h1[:, :F]) * h1[:, F:]) @ w2.t()
    return ref.dense_moe_reference(x.float(), idx, w, fn)


def _ll_worker(rank, world, port, q):
    try:
        if world > 1:
            os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
            dist.init_process_group("gloo", rank=rank, world_size=world)
        T, H, F, E, K = 24, 256, 128, 8, 3
        el = E // world
        allw = _experts(E, F, H, seed=1)
        sh = _experts(1, F, H, seed=2)
        mine = [torch.cat((s, a[rank * el:(rank + 1) * el])) for s, a in zip(sh, allw)]
        ffn = GroupedFfn(*mine, backend="bf16_bmm", bmm_cap=world * T)
        layer = NcclLowLatencyMoe(None, E, K, ffn, shared_first=True)
        x, idx, w = _inputs(rank, T, H, E, K)
        out, share = layer(x, idx, w)
        want = _dense(x, idx, w, allw, F)
        want_sh = _dense(x, torch.zeros(T, 1, dtype=torch.int64), torch.ones(T, 1), sh, F)
        e1 = ref.mean_rel_err(out.float(), want)
        e2 = ref.mean_rel_err(share.float(), want_sh)
        assert e1 < 0.02 and e2 < 0.02, (e1, e2)
        # normal mode with identity * (e + 1) experts
        ep = NcclEp(None, E)
        h = ep.prepare(idx)
        rq, rs = ep.dispatch(x, h, quant=True)
        le = torch.repeat_interleave(torch.arange(el), h["counts"])
        y = (ref.dequant_fp8_1x128(rq, rs) * (le + rank * el + 1).float().unsqueeze(1)).to(torch.bfloat16)
        res = ep.combine(y, h, ep.exchange_weights(w, h), w)
        want_n = ref.dense_moe_reference(x.float(), idx, w, lambda e, rows: rows * (e + 1))
        e3 = ref.mean_rel_err(res.float(), want_n)
        assert e3 < 0.03, e3
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()))


@pytest.mark.parametrize("world", [1, 2])
def test_baseline_layer_and_dispatch_combine_match_the_dense_oracle(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ll_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    assert all(r[1] == "ok" for r in res), res
