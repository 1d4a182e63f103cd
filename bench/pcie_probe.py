#!/usr/bin/env python
"""What the box gives N GPUs that read pinned host memory AT THE SAME TIME, measured two ways on the same pool:

  memcpy   plain cudaMemcpyAsync host -> device of 302 MB (one decode step's worth of selected KV rows) out of a pool
           allocated exactly as KvOffloadManager allocates the offloaded KV (after binding the process to the GPU's
           NUMA node), every rank at once
  gather   kv_gather_rows_kernel on the benchmark shape (batch 64, context 32768, top-2048, half the pages on the
           host), every rank at once

Run: python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/pcie_probe.py
Rank 0 prints one JSON line per method with the per-rank GB/s (device-timed with CUDA events between barriers). If
the copy engine is no faster than the gather kernel under the same N-way load, the rate is the box's ceiling (GPU
pairs share a PCIe switch uplink), not the kernel's.
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    from umdk_b200.utils.affinity import bind_to_gpu
    cpus = bind_to_gpu(local)
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from umdk_b200.ops.attention import DIM, PAGE
    from umdk_b200.ops.kv_offload import KvOffloadManager
    B, ctx, topk = 64, 32768, 2048
    P = ctx // PAGE
    half = P // 2
    kvm = KvOffloadManager(PAGE * DIM * 2, B * half, channels=1)
    pool = kvm.host_pool_tensor()
    pool[:] = 1.0
    nbytes = 302 * 1000 * 1000 // (PAGE * DIM * 2) * (PAGE * DIM * 2)
    src = pool.view(torch.uint8).reshape(-1)[:nbytes]
    dst = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    host_tab = torch.full((B, P), -1, dtype=torch.int32)
    for b in range(B):
        host_tab[b, half:] = b * half + torch.arange(half)
    host_tab = host_tab.cuda()
    idx = torch.stack([torch.randperm(ctx, device="cuda")[:topk] for _ in range(B)]).to(torch.int32)
    landing = torch.empty(B * topk, DIM, dtype=torch.bfloat16, device="cuda")
    remap = torch.empty_like(idx)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    n_host = int((idx >= half * PAGE).sum())

    def gather():
        kvm.prefetch_rows(0, idx, host_tab, landing, remap, P * PAGE, PAGE, status=status, num_ctas=8)
        kvm.wait(0)

    def timed(fn, iters=5):
        best = []
        for i in range(iters + 1):
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i > 0:
                best.append(e0.elapsed_time(e1) * 1e-3)
        best.sort()
        return best[len(best) // 2]

    res = {}
    for name, fn, nb in (("memcpy", lambda: dst.copy_(src, non_blocking=True), nbytes),
                         ("gather", gather, n_host * DIM * 2)):
        t = timed(fn)
        g = torch.tensor([nb / t / 1e9], dtype=torch.float64, device="cuda")
        if world > 1:
            allg = [torch.zeros_like(g) for _ in range(world)]
            dist.all_gather(allg, g)
            rates = [float(x) for x in allg]
        else:
            rates = [float(g)]
        res[name] = rates
        if rank == 0:
            print(json.dumps({"probe": "pcie_" + name, "n_gpus": world, "bytes_per_rank": nb,
                              "GBps_per_rank": [round(r, 1) for r in rates], "GBps_min": round(min(rates), 1),
                              "GBps_sum": round(sum(rates), 1),
                              "cpu_affinity": f"{len(cpus)} CPUs local to the GPU" if cpus else "unchanged"}), flush=True)
    assert status.tolist()[0] == 0
    kvm.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
