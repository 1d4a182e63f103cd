#!/usr/bin/env python
"""Tensor-parallel benchmarks (torchrun, one rank per GPU): Llama-style MLP, hidden 8192, FFN 28672, 8192 tokens per
step, bf16. all-gather -> GEMM for the up/gate projection, GEMM -> reduce-scatter for the down projection, and an
all-reduce sweep from 1 KiB to 1 GiB. Fused kernels versus NCCL collectives + cuBLAS, device-timed, max over ranks.
Roofline of a fused op = max(FLOPs / measured bf16 GEMM peak, NVLink bytes per rank / 770 GB/s)."""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from bench.ep_bench import emit, setup, timed  # noqa: E402

NVLINK_GBS = 770.0
BF16_TFLOPS = 1602.6


def bench_mlp(rank, world, a):
    from umdk_b200.ops.tp import TpComm
    from umdk_b200.parallel.symm import SymmetricHeap
    hidden, ffn, tokens = 8192, 28672, a.tokens
    Ts = tokens // world
    n_up = 2 * ffn // world     # gate + up columns of this rank
    k_dn = ffn // world
    g = torch.Generator(device="cuda").manual_seed(rank)
    x = torch.randn(Ts, hidden, device="cuda", generator=g).to(torch.bfloat16)
    w_up = (torch.randn(n_up, hidden, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    w_dn = (torch.randn(hidden, k_dn, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    h = torch.randn(tokens, k_dn, device="cuda", generator=g).to(torch.bfloat16)
    nbytes = TpComm.heap_bytes(world, Ts, hidden, hidden)
    heap = SymmetricHeap(nbytes, None) if world > 1 else SymmetricHeap(nbytes)
    tp = TpComm(heap, Ts, hidden, hidden, n_copy=a.n_copy)
    y = torch.empty(tokens, n_up, dtype=torch.bfloat16, device="cuda")
    o = torch.empty(Ts, hidden, dtype=torch.bfloat16, device="cuda")
    t_ag = timed(lambda: tp.ag_gemm(x, w_up, out=y), a.iters, a.warmup, world)
    t_rs = timed(lambda: tp.gemm_rs(h, w_dn, out=o), a.iters, a.warmup, world)
    tp.check()
    fl_ag, fl_rs = 2.0 * tokens * n_up * hidden, 2.0 * tokens * hidden * k_dn
    wire = (world - 1) * Ts * hidden * 2
    roof_ag = max(fl_ag / (BF16_TFLOPS * 1e12), wire / (NVLINK_GBS * 1e9))
    roof_rs = max(fl_rs / (BF16_TFLOPS * 1e12), wire / (NVLINK_GBS * 1e9))
    common = {"config": "tp_mlp", "n_gpus": world, "tokens": tokens, "hidden": hidden, "ffn": ffn}
    emit(rank, dict(common, impl="umdk_b200", op="all-gather->GEMM (up/gate)", us=t_ag * 1e6,
                    TFLOPs=fl_ag / t_ag / 1e12, roofline_us=roof_ag * 1e6, frac_of_roofline=roof_ag / t_ag))
    emit(rank, dict(common, impl="umdk_b200", op="GEMM->reduce-scatter (down)", us=t_rs * 1e6,
                    TFLOPs=fl_rs / t_rs / 1e12, roofline_us=roof_rs * 1e6, frac_of_roofline=roof_rs / t_rs))
    # baseline
    xg = torch.empty(tokens, hidden, dtype=torch.bfloat16, device="cuda")
    part = torch.empty(tokens, hidden, dtype=torch.bfloat16, device="cuda")

    def base_ag():
        if world > 1:
            dist.all_gather_into_tensor(xg, x)
        else:
            xg.copy_(x)
        torch.matmul(xg, w_up.t(), out=y)

    def base_rs():
        torch.matmul(h, w_dn.t(), out=part)
        if world > 1:
            dist.reduce_scatter_tensor(o, part)
        else:
            o.copy_(part)
    tb_ag = timed(base_ag, a.iters, a.warmup, world)
    tb_rs = timed(base_rs, a.iters, a.warmup, world)
    emit(rank, dict(common, impl="nccl_cublas_baseline", op="all_gather_into_tensor + cuBLAS", us=tb_ag * 1e6,
                    TFLOPs=fl_ag / tb_ag / 1e12, speedup_of_umdk=tb_ag / t_ag))
    emit(rank, dict(common, impl="nccl_cublas_baseline", op="cuBLAS + reduce_scatter_tensor", us=tb_rs * 1e6,
                    TFLOPs=fl_rs / tb_rs / 1e12, speedup_of_umdk=tb_rs / t_rs))
    heap.close()


def bench_allreduce(rank, world, a):
    from umdk_b200.ops.tp import AllReduce
    from umdk_b200.parallel.symm import SymmetricHeap
    max_bytes = a.max_bytes
    nbytes = AllReduce.heap_bytes(2 * max_bytes, world)   # the store-only variant stages into a second message-size area
    heap, nvls = None, False
    if world > 1 and not a.no_nvls:
        try:
            heap = SymmetricHeap.multicast(nbytes, None)
            nvls = True
        except Exception as e:  # no multicast support: peer pointers only
            if rank == 0:
                print(f"# NVLS heap unavailable ({e}); using CUDA IPC heap", flush=True)
    if heap is None:
        heap = SymmetricHeap(nbytes, None) if world > 1 else SymmetricHeap(nbytes)
    ar = AllReduce(heap, 2 * max_bytes)
    size = 1024
    while size <= max_bytes:
        n = max(size // 2, 8 * world)
        n = n // (8 * world) * (8 * world)
        x = torch.randn(n, device="cuda").to(torch.bfloat16)
        out = torch.empty_like(x)
        iters = a.iters if size <= (64 << 20) else max(3, a.iters // 4)
        res = {}
        for algo in ("one_shot", "two_shot"):
            if algo == "one_shot" and size > (8 << 20):
                continue
            res[algo] = timed(lambda: ar(x, out=out, algo=algo), iters, a.warmup, world)
        if 2 * n * world <= 2 * max_bytes and size <= (8 << 20):
            res["one_shot_push"] = timed(lambda: ar(x, out=out, algo="one_shot_push"), iters, a.warmup, world)
        if size >= (256 << 10):
            res["push"] = timed(lambda: ar(x, out=out, algo="push"), iters, a.warmup, world)
        if nvls:
            res["nvls"] = timed(lambda: ar(x, out=out, algo="nvls"), iters, a.warmup, world)
            # caller keeps its tensor in the symmetric heap: no copy in, no copy out
            res["nvls_in_place"] = timed(lambda: ar(None, algo="nvls", in_place=True, n=n), iters, a.warmup, world)
        ar.check()
        tb = timed(lambda: dist.all_reduce(out) if world > 1 else out.copy_(x), iters, a.warmup, world)
        best = min(res, key=res.get)
        bus = lambda t: 2.0 * (world - 1) / world * n * 2 / t / 1e9
        emit(rank, {"config": "allreduce", "n_gpus": world, "bytes": n * 2, "impl": "umdk_b200", "best_algo": best,
                    "us": res[best] * 1e6, "us_one_shot": res.get("one_shot", 0) * 1e6 or None,
                    "us_two_shot": res["two_shot"] * 1e6, "us_push": res.get("push", 0) * 1e6 or None, "us_one_shot_push": res.get("one_shot_push", 0) * 1e6 or None, "us_nvls": res.get("nvls", 0) * 1e6 or None,
                    "us_nvls_in_place": res.get("nvls_in_place", 0) * 1e6 or None, "bus_GBps": bus(res[best]),
                    "nccl_us": tb * 1e6, "nccl_bus_GBps": bus(tb), "speedup_vs_nccl": tb / res[best]})
        size *= 4
    heap.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["mlp", "allreduce", "all"])
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--n-copy", type=int, default=0, help="copy CTAs of all-gather -> GEMM; 0 = the default (16)")
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--no-nvls", action="store_true")
    a = ap.parse_args()
    rank, world = setup()
    if a.what in ("mlp", "all"):
        bench_mlp(rank, world, a)
    if a.what in ("allreduce", "all"):
        bench_allreduce(rank, world, a)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
