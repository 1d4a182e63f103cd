#!/usr/bin/env python
"""Expert-parallel benchmarks (run under torchrun, one rank per GPU; also works with a single process):

  normal   EP dispatch + combine, 4096 tokens/rank, hidden 7168, 256 experts top-8, fp8-e4m3 dispatch with fp32
           scales per 1x128 block, bf16 combine with top-8 weighted sum, identity experts
  ll       low-latency fused MoE layer: 128 tokens/rank, 256 experts top-8 + 1 shared expert, SwiGLU 7168->2048->7168
           with fp8-e4m3 weights and 128x128 block scales

Each prints one JSON line per measurement for the hand-written kernels and for the NCCL(+cuBLAS) baseline: time in
microseconds (device-timed with CUDA events, max over ranks, 256 MB L2 flush between iterations), GB/s of received
bytes, and the fraction of the NVLink roofline (bytes that must cross NVLink per rank / 770 GB/s measured peer-copy
bandwidth). Same measurement shape as the reference's sample (src/cam/examples/moe_dispatch_combine_prefill_sample.py:
213-267: warm-up + timed iterations, L2 flush, GB/s = received bytes / time).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

NVLINK_GBS = 770.0
HBM_GBS = 6553.0


def setup():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world


_flush = None


def timed(fn, iters, warmup, world):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    tot = 0.0
    for _ in range(iters):
        _flush.zero_()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # the GPU idles ~100 us while the host queues the call: the events then bracket device time, not the time
        # the Python wrapper needs to launch
        torch.cuda._sleep(200000)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e1)
    t = torch.tensor([tot / iters], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) * 1e-3  # seconds


_records = []
_quiet = False


def emit(rank, rec):
    _records.append(rec)
    if rank == 0 and not _quiet:
        print(json.dumps(rec), flush=True)


def _begin(quiet):
    global _quiet
    _quiet = quiet
    _records.clear()


def routing(T, E, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    logits = torch.randn(T, E, device="cuda", generator=g)
    p = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(p, K, dim=-1)
    return idx.to(torch.int64).contiguous(), (w / w.sum(-1, keepdim=True)).float().contiguous()


def bench_normal(rank, world, a, quiet=False):
    """Returns the list of records it emitted (every rank gets the same list; rank 0 prints unless ``quiet``)."""
    from baseline.nccl_baseline import NcclEp
    _begin(quiet)
    brief = getattr(a, "brief", False)
    from umdk_b200.ops.ep import EpNormal
    from umdk_b200.parallel.symm import SymmetricHeap
    T, H, E, K = a.tokens, 7168, 256, 8
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    idx, w = routing(T, E, K, 200 + rank)
    nbytes = EpNormal.heap_bytes(world, E, K, H, T)
    heap = SymmetricHeap(nbytes, None) if world > 1 else SymmetricHeap(nbytes)
    st = EpNormal(heap, E, K, H, T)
    lay = st.layout(idx)
    out = st.dispatch(x, idx, w, lay=lay, quant=True, sync_counts=True)
    n = out.num_recv
    arrivals = int(out.counts[1].item())
    y = torch.randn(out.recv_x.shape[0], H, device="cuda").to(torch.bfloat16)
    res = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    remote_frac = (world - 1) / world
    t_lay = timed(lambda: st.layout(idx, out=lay), a.iters, a.warmup, world)
    t_disp = timed(lambda: st.dispatch(x, idx, w, lay=lay, quant=True, out=out), a.iters, a.warmup, world)
    t_comb = timed(lambda: st.combine(y, out, out=res), a.iters, a.warmup, world)
    st.check("normal")
    waits = None
    if not brief:
        # diagnose mode: how long CTA 0 of this rank waited for each source rank's data (max over ranks per source)
        st.diagnose = True
        st.dispatch(x, idx, w, lay=lay, quant=True, out=out)
        st.combine(y, out, out=res)
        torch.cuda.synchronize()
        wd, wc = st.wait_times_us()
        st.diagnose = False
        waits = torch.stack((wd, wc)).cuda()
        if world > 1:
            dist.all_reduce(waits, op=dist.ReduceOp.MAX)
        waits = waits.cpu()
    row_b = H + H // 32
    wire_d = arrivals * row_b * remote_frac          # each token crosses once per destination rank
    wire_c = arrivals * H * 2 * remote_frac
    common = {"config": "ep_normal", "n_gpus": world, "tokens_per_rank": T, "hidden": H, "experts": E, "top_k": K,
              "impl": "umdk_b200"}
    emit(rank, dict(common, op="layout", us=t_lay * 1e6))
    emit(rank, dict(common, op="dispatch(fp8 1x128)", us=t_disp * 1e6, recv_rows=n, arrivals=arrivals,
                    recv_GBps=n * row_b / t_disp / 1e9, nvlink_GBps=wire_d / t_disp / 1e9,
                    frac_of_nvlink_roofline=(wire_d / (NVLINK_GBS * 1e9)) / t_disp if world > 1 else None,
                    frac_of_hbm_roofline=((T * H * 2 + 2 * arrivals * row_b + n * row_b) / (HBM_GBS * 1e9)) / t_disp))
    emit(rank, dict(common, op="combine(bf16, top-8 weighted)", us=t_comb * 1e6,
                    recv_GBps=n * H * 2 / t_comb / 1e9, nvlink_GBps=wire_c / t_comb / 1e9,
                    frac_of_nvlink_roofline=(wire_c / (NVLINK_GBS * 1e9)) / t_comb if world > 1 else None))
    if waits is not None:
        emit(rank, dict(common, op="diagnose: wait per source rank (us, max over ranks)",
                        dispatch=[round(float(v), 1) for v in waits[0]], combine=[round(float(v), 1) for v in waits[1]]))
    # baseline: one row per (token, rank) over all_to_all_single, index work and split sizes prepared outside the
    # timed call (as the product's layout is); plus the collective alone on the same bytes
    base = NcclEp(None, E)
    h = base.prepare(idx)
    wrecv = base.exchange_weights(w, h)
    rq, _ = base.dispatch(x, h, True)
    yb = torch.randn(rq.shape[0], H, device="cuda").to(torch.bfloat16)
    tb_d = timed(lambda: base.dispatch(x, h, True), a.iters, a.warmup, world)
    tb_c = timed(lambda: base.combine(yb, h, wrecv, w), a.iters, a.warmup, world)
    tw_d = timed(base.bare_all_to_all(h, row_b), a.iters, a.warmup, world)
    tw_c = timed(base.bare_all_to_all(h, 2 * H, reverse=True), a.iters, a.warmup, world)
    emit(rank, dict(common, impl="nccl_baseline", op="dispatch(fp8 1x128)", us=tb_d * 1e6,
                    recv_GBps=rq.shape[0] * row_b / tb_d / 1e9, speedup_of_umdk=tb_d / t_disp))
    emit(rank, dict(common, impl="nccl_baseline", op="combine(bf16, top-8 weighted)", us=tb_c * 1e6,
                    speedup_of_umdk=tb_c / t_comb))
    emit(rank, dict(common, impl="nccl_baseline", op="bare all_to_all_single, dispatch bytes", us=tw_d * 1e6))
    emit(rank, dict(common, impl="nccl_baseline", op="bare all_to_all_single, combine bytes", us=tw_c * 1e6))
    heap.close()
    return list(_records)


def bench_ll(rank, world, a, quiet=False):
    from baseline.nccl_baseline import GroupedFfn, NcclLowLatencyMoe
    from umdk_b200.models.dsv3_decoder import _quant_experts
    from umdk_b200.ops.ep_ll import EpLowLatency, ExpertWeights
    from umdk_b200.parallel.symm import SymmetricHeap
    _begin(quiet)
    brief = getattr(a, "brief", False)
    T, H, F, E, K = a.ll_tokens, 7168, 2048, a.ll_experts, 8
    el = E // world
    g = torch.Generator(device="cuda").manual_seed(300 + rank)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    idx, w = routing(T, E, K, 400 + rank)
    w1q, w1s = _quant_experts(el, 2 * F, H, "cuda", g)
    w2q, w2s = _quant_experts(el, H, F, "cuda", g)
    s1q, s1s = _quant_experts(1, 2 * F, H, "cuda", g)
    s2q, s2s = _quant_experts(1, H, F, "cuda", g)
    experts, shared = ExpertWeights(w1q, w1s, w2q, w2s), ExpertWeights(s1q, s1s, s2q, s2s)
    nbytes = EpLowLatency.heap_bytes(world, E, K, H, T)
    heap = SymmetricHeap(nbytes, None) if world > 1 else SymmetricHeap(nbytes)
    ll = EpLowLatency(heap, E, K, H, F, T)
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    tiled = experts.to_tiled()
    t_tiled = timed(lambda: ll.moe(x, idx, w, tiled, None, out=out), a.iters, a.warmup, world)
    ll.check("ll")
    rows = int(ll.group_off[-1].item())
    w_bytes = (w1q.numel() + w2q.numel())              # routed expert weights read once per call
    flops = 2.0 * rows * (2 * F * H + H * F)
    wire = (T * K * (H + H // 32) + T * K * H * 2) * (world - 1) / world
    roof = max(w_bytes / (HBM_GBS * 1e9), flops / (2 * 1602.6e12), wire / (NVLINK_GBS * 1e9))
    common = {"config": "ep_ll_moe", "n_gpus": world, "tokens_per_rank": T, "hidden": H, "ffn": F, "experts": E,
              "top_k": K, "rows_on_this_rank": rows}
    rec_tiled = dict(common, impl="umdk_b200", op="routed only, tile-major weights (ExpertWeights.to_tiled)",
                     us=t_tiled * 1e6, roofline_us=roof * 1e6, frac_of_roofline=roof / t_tiled,
                     weight_GBps=w_bytes / t_tiled / 1e9)
    if not brief:
        t_all = timed(lambda: ll.moe(x, idx, w, experts, shared, out=out), a.iters, a.warmup, world)
        t_routed = timed(lambda: ll.moe(x, idx, w, experts, None, out=out), a.iters, a.warmup, world)
        t_two = timed(lambda: ll.moe(x, idx, w, experts, None, out=out, fused=False), a.iters, a.warmup, world)
        # inside the fused kernel: global-timer stamps of its stages (median of 5 calls, max over ranks)
        ll.diagnose = True
        tls = []
        for _ in range(5):
            ll.timeline_reset()
            ll.moe(x, idx, w, tiled, None, out=out)
            torch.cuda.synchronize()
            tls.append(list(ll.timeline_us().values()))
        ll.diagnose = False
        tl = torch.tensor(tls, dtype=torch.float64).median(dim=0).values.cuda()
        if world > 1:
            dist.all_reduce(tl, op=dist.ReduceOp.MAX)
        rec_tiled["fused_timeline_us"] = dict(zip(ll.timeline_names(), [round(float(v), 1) for v in tl]))
        emit(rank, dict(common, impl="umdk_b200", op="dispatch+GEMM1+SwiGLU+quant+GEMM2+combine (+shared expert)",
                        us=t_all * 1e6))
        emit(rank, dict(common, impl="umdk_b200", op="dispatch+GEMM1+SwiGLU+quant+GEMM2+combine (routed only)",
                        us=t_routed * 1e6, roofline_us=roof * 1e6, frac_of_roofline=roof / t_routed,
                        weight_GBps=w_bytes / t_routed / 1e9))
        emit(rank, dict(common, impl="umdk_b200", op="same, expert GEMMs as two launches (moe_gemm mode 0 + mode 2)",
                        us=t_two * 1e6, frac_of_roofline=roof / t_two))
    emit(rank, rec_tiled)
    if not brief:
        # the same layer as one CUDA-graph replay: no Python / launch cost between the kernels
        try:
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            graph, _ = ll.capture(x, idx, w, tiled, None, out=out)
            t_graph = timed(graph.replay, a.iters, a.warmup, world)
            ll.check("ll graph")
            del graph
            emit(rank, dict(common, impl="umdk_b200", op="routed only, tile-major weights, one CUDA-graph replay per layer",
                            us=t_graph * 1e6, frac_of_roofline=roof / t_graph, weight_GBps=w_bytes / t_graph / 1e9))
        except Exception as e:  # capture not possible in this environment: report without it
            if rank == 0:
                print(f"# CUDA graph capture of the layer failed: {e}", flush=True)
    del tiled
    # baseline: all_gather + ONE grouped library GEMM per projection + reduce_scatter, no host synchronisation
    ffn = GroupedFfn(w1q, w1s, w2q, w2s, bmm_cap=world * T)
    base = NcclLowLatencyMoe(None, E, K, ffn, shared_first=False)
    tb = timed(lambda: base(x, idx, w), a.iters, a.warmup, world)
    emit(rank, dict(common, impl="nccl_grouped_gemm_baseline", gemm=ffn.backend,
                    op="all_gather + grouped library GEMMs (" + ffn.backend + ") + reduce_scatter",
                    us=tb * 1e6, speedup_of_umdk=tb / t_tiled))
    heap.close()
    return list(_records)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["normal", "ll", "all"])
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--ll-tokens", type=int, default=128)
    ap.add_argument("--ll-experts", type=int, default=256,
                    help="routed experts in total; 32 on one GPU is the share of one rank at EP = 8, without the wire")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    rank, world = setup()
    if a.what in ("normal", "all"):
        bench_normal(rank, world, a)
    if a.what in ("ll", "all"):
        bench_ll(rank, world, a)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
