"""Helpers shared by the example programs: process-group bootstrap, device-side timing with an L2 flush between
iterations, per-kernel timing through the torch profiler, and the rank x rank "slow link" diagnosis.

Counterpart of the reference's example helpers (src/cam/examples/utils.py:38-47 init_dist, :67-101 bench,
:104-198 bench_kineto, :297-341 diagnose_matrix), written against torch.distributed/NCCL and CUDA events.
"""
from __future__ import annotations

import os
import sys
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def init_dist(backend: Optional[str] = None) -> Tuple[int, int, Optional[dist.ProcessGroup]]:
    """Reads RANK / WORLD_SIZE / LOCAL_RANK (torchrun) and initialises the default group.
    Returns (rank, world, group); a single process without the variables runs as world 1 without a group."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local)
    if world == 1:
        return 0, 1, None
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29555")
    backend = backend or ("nccl" if use_cuda else "gloo")
    kw = {"device_id": torch.device("cuda", local)} if backend == "nccl" else {}
    dist.init_process_group(backend, rank=rank, world_size=world, **kw)
    return rank, world, dist.group.WORLD


_flush_buf = None


def bench(fn: Callable[[], object], num_warmups: int = 50, num_tests: int = 50, flush_l2: bool = True
          ) -> Tuple[float, float, float]:
    """(avg, min, max) seconds of fn() on the current stream, CUDA-event timed; 256 MB are written between
    iterations so that no input is served from L2."""
    global _flush_buf
    if flush_l2 and _flush_buf is None:
        _flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(num_warmups):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(num_tests):
        if flush_l2:
            _flush_buf.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    return sum(ts) / len(ts), min(ts), max(ts)


def bench_kineto(fn: Callable[[], object], kernel_names: List[str], num_tests: int = 20, barrier: bool = True
                 ) -> List[float]:
    """Average device time (seconds) of the kernels whose name contains each entry of kernel_names, taken from a
    torch profiler trace of num_tests calls."""
    from torch.profiler import ProfilerActivity, profile
    fn()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(num_tests):
            if barrier and dist.is_initialized():
                dist.barrier()
            fn()
        torch.cuda.synchronize()
    out = []
    for name in kernel_names:
        tot, cnt = 0.0, 0
        for ev in prof.key_averages():
            if name in ev.key:
                tot += ev.device_time_total
                cnt += ev.count
        out.append(tot / max(cnt, 1) * 1e-6)
    return out


def diagnose_matrix(times_us: torch.Tensor, thres_col: float = 3.0, thres_row: float = 3.0,
                    thres_point: float = 5.0) -> dict:
    """times_us[src, dst]: waiting time one rank observed for another. Flags columns / rows / single entries whose
    value exceeds the given multiple of the matrix mean - a slow destination, a slow source, or one bad link."""
    m = times_us.double()
    mean = m.mean().clamp_min(1e-9)
    cols = (m.mean(dim=0) > thres_col * mean).nonzero().flatten().tolist()
    rows = (m.mean(dim=1) > thres_row * mean).nonzero().flatten().tolist()
    pts = [(int(i), int(j)) for i, j in (m > thres_point * mean).nonzero().tolist()
           if int(i) not in rows and int(j) not in cols]
    return {"mean_us": float(mean), "abnormal_cols": cols, "abnormal_rows": rows, "abnormal_points": pts}


def gather_matrix(row: torch.Tensor, group=None) -> Optional[torch.Tensor]:
    """Every rank contributes one row [world]; rank 0 gets the [world, world] matrix (others None)."""
    if not dist.is_initialized():
        return row.reshape(1, -1).cpu()
    world = dist.get_world_size(group)
    rows = [torch.empty_like(row) for _ in range(world)]
    dist.all_gather(rows, row, group=group)
    return torch.stack(rows).cpu() if dist.get_rank(group) == 0 else None


def routing(tokens: int, num_experts: int, top_k: int, seed: int, device="cpu"):
    """top-k routing from N(0,1) gate logits with softmax; weights renormalised over the selected experts."""
    g = torch.Generator().manual_seed(seed)
    p = torch.softmax(torch.randn(tokens, num_experts, generator=g), dim=-1)
    w, idx = torch.topk(p, top_k, dim=-1)
    return idx.to(torch.int64).to(device), (w / w.sum(-1, keepdim=True)).float().to(device)
