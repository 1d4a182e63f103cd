#!/usr/bin/env python
"""Single-GPU timing of the individual hand-written kernels with their roofline fractions.

    python bench/kernel_bench.py moe_gemm1 --tokens-per-expert 32 --experts 32
    python bench/kernel_bench.py moe_gemm2 | mla | dispatch | combine | gemm_bf16 | quant | all

Timing hygiene: >= 3 warm-up launches, an L2 flush (256 MB write) before every timed launch, CUDA events on the
launching stream. The same role as the reference's `bench()` helper (src/cam/examples/utils.py:67-101: 256 MB L2
flush, event timing). Roofline denominators come from MEASURED_PEAKS.json at the repo root when present
(6553 GB/s copy bandwidth, 1602.6 TFLOP/s bf16 burst), otherwise the fallback 6650 GB/s / 1590 TFLOP/s.
`--small` shrinks a case so that a profiler capture of it stays short.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from umdk_b200.ops import reference as ref  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def time_kernel(fn, iters=10, warmup=3):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # keep the GPU busy for ~100 us while the host queues the call, so that the interval between the two events
        # is the kernel and not the time the Python wrapper needs to launch it
        torch.cuda._sleep(200000)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2] * 1e-3, ts[0] * 1e-3


def report(name, sec_med, sec_min, bytes_, flops, extra=None):
    hbm, tf, how = peaks()
    gbs = bytes_ / sec_med / 1e9
    tfl = flops / sec_med / 1e12
    t_roof = max(bytes_ / (hbm * 1e9), flops / (tf * 1e12))
    out = {"kernel": name, "us": sec_med * 1e6, "us_min": sec_min * 1e6, "GB/s": gbs, "TFLOP/s": tfl,
           "frac_of_hbm_" + how: gbs / hbm, "frac_of_bf16_" + how: tfl / tf, "roofline_us": t_roof * 1e6,
           "frac_of_roofline": t_roof / sec_med}
    if extra:
        out.update(extra)
    print(json.dumps(out), flush=True)
    return out


def _rand_fp8(*shape):
    # random e4m3 payload in [-1.75, 1.75] without going through a large fp32 tensor
    b = torch.randint(0, 0x40, shape, dtype=torch.uint8, device="cuda")
    b |= (torch.randint(0, 2, shape, dtype=torch.uint8, device="cuda") << 7)
    return b.view(torch.float8_e4m3fn)


def bench_moe_gemm(which, experts, tpe, H=7168, F=2048):
    from umdk_b200.ops import moe_gemm
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    N = experts * tpe
    off = (torch.arange(experts + 1, dtype=torch.int32) * tpe).cuda()
    if which == 1:
        xq, xs = _rand_fp8(N, H), torch.rand(N, H // 128, device="cuda") * 0.01 + 0.005
        wq, ws = _rand_fp8(experts, 2 * F, H), torch.rand(experts, 2 * F // 128, H // 128, device="cuda") * 0.01
        hq = torch.empty(N, F, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
        hs = torch.empty(N, F // 128, dtype=torch.float32, device="cuda")
        fn = lambda: moe_gemm.gemm1_swiglu_quant(xq, xs, off, wq, ws, status, hq, hs)
        bytes_ = wq.numel() + ws.numel() * 4 + xq.numel() + xs.numel() * 4 + hq.numel() + hs.numel() * 4
        flops = 2.0 * N * 2 * F * H
        name = "moe_gemm_mode0(gate/up+SwiGLU+requant)"
    else:
        xq, xs = _rand_fp8(N, F), torch.rand(N, F // 128, device="cuda") * 0.01 + 0.005
        wq, ws = _rand_fp8(experts, H, F), torch.rand(experts, H // 128, F // 128, device="cuda") * 0.01
        y = torch.empty(N, H, dtype=torch.bfloat16, device="cuda")
        fn = lambda: moe_gemm.gemm2(xq, xs, off, wq, ws, status, y)
        bytes_ = wq.numel() + ws.numel() * 4 + xq.numel() + xs.numel() * 4 + y.numel() * 2
        flops = 2.0 * N * H * F
        name = "moe_gemm_mode1(down)"
    med, mn = time_kernel(fn)
    assert status.tolist()[0] == 0, status.tolist()
    return report(name, med, mn, bytes_, flops, {"experts": experts, "tokens_per_expert": tpe, "H": H, "F": F})


def bench_mla(B, ctx, topk):
    from umdk_b200.ops.attention import DIM, HEADS, PAGE, sparse_mla_decode
    pps = ctx // PAGE
    kv = (torch.randn(B * pps, PAGE, DIM, device="cuda") * 0.5).to(torch.bfloat16)
    bt = torch.arange(B * pps, dtype=torch.int32, device="cuda").reshape(B, pps)
    q = (torch.randn(B, HEADS, DIM, device="cuda") * 0.5).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(ctx, device="cuda")[:topk] for _ in range(B)]).to(torch.int32)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.empty(B, HEADS, 512, dtype=torch.bfloat16, device="cuda")
    fn = lambda: sparse_mla_decode(q, kv, bt, idx, DIM ** -0.5, out=out, status=status)
    med, mn = time_kernel(fn)
    assert status.tolist()[0] == 0
    bytes_ = B * topk * DIM * 2 + q.numel() * 2 + out.numel() * 2
    flops = 2.0 * B * HEADS * topk * (DIM + 512)
    return report("sparse_mla_decode", med, mn, bytes_, flops, {"B": B, "ctx": ctx, "topk": topk})


def bench_moe_fused(experts, tokens, H=7168, F=2048, K=8, tiled=True):
    """The low-latency MoE layer at EP = 1 (dispatch + fused expert kernel): every token stays on this GPU, so the
    NVLink stores of the combine epilogue land in local memory."""
    from umdk_b200.models.dsv3_decoder import _quant_experts
    from umdk_b200.ops.ep_ll import EpLowLatency, ExpertWeights
    from umdk_b200.parallel.symm import SymmetricHeap
    g = torch.Generator(device="cuda").manual_seed(3)
    K = min(K, experts)
    x = torch.randn(tokens, H, device="cuda", generator=g).to(torch.bfloat16)
    p = torch.softmax(torch.randn(tokens, experts, device="cuda", generator=g), dim=-1)
    w, idx = torch.topk(p, K, dim=-1)
    w = (w / w.sum(-1, keepdim=True)).float().contiguous()
    idx = idx.to(torch.int64).contiguous()
    ew = ExpertWeights(*_quant_experts(experts, 2 * F, H, "cuda", g), *_quant_experts(experts, H, F, "cuda", g))
    if tiled:
        ew = ew.to_tiled()
    heap = SymmetricHeap(EpLowLatency.heap_bytes(1, experts, K, H, tokens))
    ll = EpLowLatency(heap, experts, K, H, F, tokens)
    out = torch.empty(tokens, H, dtype=torch.bfloat16, device="cuda")
    med, mn = time_kernel(lambda: ll.moe(x, idx, w, ew, None, out=out))
    ll.check("moe_fused")
    bytes_ = experts * 3 * F * H
    flops = 2.0 * tokens * K * 3 * F * H
    r = report("ep_layout + ep_ll_dispatch + moe_fused (EP=1)", med, mn, bytes_, flops,
               {"experts": experts, "tokens": tokens, "top_k": K, "H": H, "F": F, "tile_major_weights": tiled})
    heap.close()
    return r


def bench_tp_loopback(Ts, K, N):
    """Tensor-parallel fused kernels with a single rank: the copy CTAs and the push epilogue run against this GPU's own
    heap, so this times the kernels' compute path (CTA pairs) without NVLink."""
    from umdk_b200.ops.tp import TpComm
    from umdk_b200.parallel.symm import SymmetricHeap
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(Ts, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    heap = SymmetricHeap(TpComm.heap_bytes(1, Ts, K, N))
    tp = TpComm(heap, Ts, K, N)
    out = torch.empty(Ts, N, dtype=torch.bfloat16, device="cuda")
    med, mn = time_kernel(lambda: tp.ag_gemm(x, w, out=out))
    tp.check()
    report("tp all-gather->GEMM, 1 rank (CTA pairs)", med, mn, (Ts * K + N * K + Ts * N) * 2, 2.0 * Ts * N * K,
           {"Ts": Ts, "K": K, "N": N})
    med, mn = time_kernel(lambda: tp.gemm_rs(x, w, out=out))
    tp.check()
    r = report("tp GEMM->reduce-scatter, 1 rank (CTA pairs)", med, mn, (Ts * K + N * K + 3 * Ts * N) * 2,
               2.0 * Ts * N * K, {"Ts": Ts, "K": K, "N": N})
    heap.close()
    return r


def bench_kv_gather(B, ctx, topk, num_ctas=8):
    """Row-granular KV prefetch: rows of the offloaded half of every sequence read straight from pinned host memory
    by the gather kernel (PCIe-bound; the HBM columns of the report do not apply)."""
    from umdk_b200.ops.attention import DIM, PAGE
    from umdk_b200.ops.kv_offload import KvOffloadManager
    P = ctx // PAGE
    half = P // 2
    kvm = KvOffloadManager(PAGE * DIM * 2, B * half, channels=1)
    kvm.host_pool_tensor()[:] = 1.0
    host_tab = torch.full((B, P), -1, dtype=torch.int32)
    for b in range(B):
        host_tab[b, half:] = b * half + torch.arange(half)
    host_tab = host_tab.cuda()
    idx = torch.stack([torch.randperm(ctx, device="cuda")[:topk] for _ in range(B)]).to(torch.int32)
    landing = torch.empty(B * topk, DIM, dtype=torch.bfloat16, device="cuda")
    remap = torch.empty_like(idx)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")

    def fn():
        kvm.prefetch_rows(0, idx, host_tab, landing, remap, P * PAGE, PAGE, status=status, num_ctas=num_ctas)
        kvm.wait(0)

    med, mn = time_kernel(fn)
    assert status.tolist()[0] == 0
    n_host = int((idx >= half * PAGE).sum())
    bytes_ = n_host * DIM * 2
    out = {"kernel": "kv_gather_rows (pinned host -> device over PCIe)", "us": med * 1e6, "us_min": mn * 1e6,
           "host_rows": n_host, "row_bytes": DIM * 2, "pcie_GB/s": bytes_ / med / 1e9, "B": B, "ctx": ctx,
           "topk": topk, "ctas_of_1024_threads": num_ctas}
    print(json.dumps(out), flush=True)
    # the same bytes as one contiguous cudaMemcpyAsync, for the PCIe ceiling of this box
    src = torch.empty(bytes_, dtype=torch.uint8).pin_memory()
    dst = torch.empty(bytes_, dtype=torch.uint8, device="cuda")
    med2, _ = time_kernel(lambda: dst.copy_(src, non_blocking=True))
    print(json.dumps({"kernel": "cudaMemcpyAsync H2D of the same byte count (ceiling)", "us": med2 * 1e6,
                      "pcie_GB/s": bytes_ / med2 / 1e9}), flush=True)
    kvm.close()
    return out


def bench_dispatch_combine(T, H, E, K):
    """World size 1: every token stays on the GPU, so this measures the kernels' local memory path only."""
    from umdk_b200.ops.ep import EpNormal
    from umdk_b200.parallel.symm import SymmetricHeap
    heap = SymmetricHeap(EpNormal.heap_bytes(1, E, K, H, T))
    st = EpNormal(heap, E, K, H, T)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    idx = torch.topk(torch.rand(T, E, device="cuda"), K, dim=-1).indices.to(torch.int64)
    w = torch.rand(T, K, device="cuda")
    lay = st.layout(idx)
    out = st.dispatch(x, idx, w, lay=lay, quant=True)
    res = []
    med, mn = time_kernel(lambda: st.layout(idx))
    res.append(report("ep_layout", med, mn, idx.numel() * 8 + T * K * 4 + T * 4, 0, {"T": T, "E": E, "K": K}))
    med, mn = time_kernel(lambda: st.dispatch(x, idx, w, lay=lay, quant=True, out=out))
    n = T * K
    bytes_ = x.numel() * 2 + 2 * T * (H + H // 32) + n * (H + H // 32)  # read x, write+read arrivals, write rows
    res.append(report("ep_dispatch(world=1)", med, mn, bytes_, 0, {"T": T, "H": H, "rows": n}))
    y = torch.randn(out.recv_x.shape[0], H, device="cuda").to(torch.bfloat16)
    o = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    med, mn = time_kernel(lambda: st.combine(y, out, out=o))
    bytes_ = n * H * 2 + 2 * T * H * 2 + T * H * 2
    res.append(report("ep_combine(world=1)", med, mn, bytes_, 0, {"T": T, "H": H, "rows": n}))
    st.check()
    heap.close()
    return res


def bench_allreduce(nbytes):
    """Two-shot all-reduce kernel with a single rank: the reduce-scatter and all-gather passes run against this
    GPU's own heap (read x, write the slice, read it back, write out), which is the kernel's memory path."""
    from umdk_b200.ops.tp import AllReduce
    from umdk_b200.parallel.symm import SymmetricHeap
    heap = SymmetricHeap(AllReduce.heap_bytes(nbytes, 1))
    ar = AllReduce(heap, nbytes)
    x = torch.randn(nbytes // 2, device="cuda").to(torch.bfloat16)
    med, mn = time_kernel(lambda: ar(x, algo="two_shot"))
    ar.check()
    r = report("allreduce two_shot (world=1)", med, mn, 4 * nbytes, 0, {"bytes": nbytes})
    heap.close()
    return r


def bench_ll_combine(T, H, E, K):
    """The stand-alone low-latency combine kernel at EP = 1: rows of the expert-major slab go back to the token
    owner's combine buffer (local stores here), flags, weighted sum."""
    from umdk_b200.ops.ep_ll import EpLowLatency
    from umdk_b200.parallel.symm import SymmetricHeap
    heap = SymmetricHeap(EpLowLatency.heap_bytes(1, E, K, H, T))
    st = EpLowLatency(heap, E, K, H, 256, T)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    idx = torch.topk(torch.rand(T, E, device="cuda"), K, dim=-1).indices.to(torch.int64)
    w = torch.rand(T, K, device="cuda")
    y = torch.randn(st.n_cap, H, device="cuda").to(torch.bfloat16)
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")

    def step():
        st.dispatch(x, idx)
        st.combine(y, idx, w, out=out)
    med, mn = time_kernel(step)
    st.check()
    n = T * K
    r = report("ep_ll_dispatch + ep_ll_combine (EP=1)", med, mn, T * H * 2 + 2 * n * H + 3 * n * H * 2 + T * H * 2, 0,
               {"T": T, "H": H, "rows": n})
    heap.close()
    return r


def bench_gemm_bf16(M, N, K):
    from umdk_b200 import _native
    lib = _native.cam()
    A = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    B = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    C = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")

    def fn():
        rc = lib.umdk_gemm_bf16(_native.ptr(A), _native.ptr(B), _native.ptr(C), M, N, K, K, K, N, _native.ptr(st),
                                _native.stream_ptr(), 0)
        assert rc == 0
    med, mn = time_kernel(fn)
    r = report("gemm_bf16_tcgen05", med, mn, (M * K + N * K + M * N) * 2, 2.0 * M * N * K, {"M": M, "N": N, "K": K})
    if M % 256 == 0 and N % 256 == 0 and K % 64 == 0:
        def fn2():
            rc = lib.umdk_gemm_bf16_2sm(_native.ptr(A), _native.ptr(B), _native.ptr(C), M, N, K, K, K, N,
                                        _native.ptr(st), _native.stream_ptr(), 0)
            assert rc == 0
        med, mn = time_kernel(fn2)
        assert st.tolist()[0] == 0, st.tolist()
        report("gemm_bf16_tcgen05_cta_pair", med, mn, (M * K + N * K + M * N) * 2, 2.0 * M * N * K,
               {"M": M, "N": N, "K": K})
    med, mn = time_kernel(lambda: torch.matmul(A, B.t(), out=C))
    report("cublas_bf16(torch.matmul)", med, mn, (M * K + N * K + M * N) * 2, 2.0 * M * N * K, {"M": M, "N": N, "K": K})
    return r


def bench_quant(T, H):
    from umdk_b200.ops.ep_ll import quant_fp8_1x128
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    med, mn = time_kernel(lambda: quant_fp8_1x128(x))
    return report("quant_fp8_1x128", med, mn, T * H * 3 + T * H // 32, 0, {"T": T, "H": H})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["moe_gemm1", "moe_gemm2", "mla", "kv_gather", "dispatch", "gemm_bf16", "quant", "moe_fused", "tp", "allreduce", "ll_combine", "all"])
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--tokens-per-expert", type=int, default=32)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--topk", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--fused-experts", type=int, default=0,
                    help="moe_fused: local experts (32 = the share of one rank at EP = 8); default 256, or 8 with --small")
    a = ap.parse_args()
    if a.small:
        a.experts, a.batch, a.ctx, a.tokens = min(a.experts, 8), min(a.batch, 16), min(a.ctx, 8192), min(a.tokens, 1024)
    if a.what in ("moe_gemm1", "all"):
        bench_moe_gemm(1, a.experts, a.tokens_per_expert)
    if a.what in ("moe_gemm2", "all"):
        bench_moe_gemm(2, a.experts, a.tokens_per_expert)
    if a.what in ("mla", "all"):
        bench_mla(a.batch, a.ctx, a.topk)
    if a.what in ("moe_fused", "all"):
        bench_moe_fused(a.fused_experts or (a.experts if a.small else 256), 128)
    if a.what in ("tp", "all"):
        bench_tp_loopback(2048, 4096, 4096) if a.small else bench_tp_loopback(8192, 8192, 7168)
    if a.what in ("kv_gather", "all"):
        for n in (4, 8, 16, 32):
            bench_kv_gather(a.batch, a.ctx, a.topk, n)
    if a.what in ("dispatch", "all"):
        bench_dispatch_combine(a.tokens, 7168, 256, 8)
    if a.what in ("gemm_bf16", "all"):
        bench_gemm_bf16(8192, 8192, 8192) if not a.small else bench_gemm_bf16(4096, 4096, 4096)
    if a.what in ("allreduce", "all"):
        bench_allreduce((256 << 20) if a.small else (1 << 30))
    if a.what in ("ll_combine", "all"):
        bench_ll_combine(128 if not a.small else 64, 7168, 256 if not a.small else 32, 8)
    if a.what in ("quant", "all"):
        bench_quant(a.tokens, 7168)


if __name__ == "__main__":
    main()
