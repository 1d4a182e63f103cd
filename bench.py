#!/usr/bin/env python
"""Flagship benchmark: MoE decode tokens/sec per box on a DeepSeek-V3-shaped 4-layer MoE decoder.

One decode step per rank = batch 64 sequences x 1 token, context 32768 in a paged bf16 MLA KV cache (64-token pages),
sparse attention over top-2048 KV rows per query chosen uniformly at random, half of every sequence's pages offloaded
to pinned host memory (cudaMemcpyAsync on a side stream) and brought back on that side stream every step - by default
only the token rows the step's indices select, gathered by a kernel that reads the pinned pool directly
(--kv-fetch rows); or every offloaded page with cudaMemcpyAsync (--kv-fetch pages) - MoE layers with 256 routed experts
(top-8, fp8 e4m3 SwiGLU experts 7168 -> 2048 -> 7168 with 128x128 block scales) plus one shared expert, experts
sharded over the N ranks (EP = N), attention data parallel (weak scaling: 64 sequences per GPU).

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 8 --warmup 3

Rank 0 prints ONE JSON line. `value` is device-timed (CUDA events, max over ranks, median of --repeats timed regions
of exactly --steps steps) with inputs resident on the device; `e2e.value` goes through the public `DecoderRank.step`
API with the step's inputs copied from pinned host memory and the sampled tokens read back on the host every step.

Because the reference project cannot run on NVIDIA GPUs, the same process first times the SAME decode step written
with PyTorch + NCCL + library GEMMs only (baseline/decode_baseline.py: torch gather + matmul attention, every
offloaded page copied back with cudaMemcpyAsync on a side stream, all_gather / grouped library GEMM / reduce_scatter
MoE) and reports `vs_baseline` = product / baseline (device-timed) and `e2e.vs_baseline`. `--impl baseline` runs that
arm alone. `extra` carries the other named sub-metrics: the product with every offloaded page prefetched
(`pages_mode`), with the whole cache resident (`compute_only`, both arms), and on 2 or more GPUs the EP normal-mode
dispatch / combine and the low-latency MoE layer with their NCCL baselines.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REFERENCE_UNAVAILABLE = ("reference is Ascend-only (AscendC kernels built with CANN/HCCL, UB kernel modules; no "
                         "setup.py/pyproject at its root: pip reports 'Neither setup.py nor pyproject.toml found'); "
                         "it cannot be built for or run on NVIDIA GPUs")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs: NVML (read-only queries) from
    a thread every 10 ms, or `nvidia-smi -lms 50` if the NVML binding is missing."""

    REASONS = ((0x4, "sw_power_cap"), (0x8, "hw_slowdown"), (0x20, "sw_thermal_slowdown"),
               (0x40, "hw_thermal_slowdown"))
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = self._physical_index(gpu_index)
        self.sm, self.mx, self.reasons, self.power = [], None, set(), []
        self._stop = threading.Event()
        self._thread = None
        self._proc = None
        self._how = None

    @staticmethod
    def _physical_index(i: int) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if i < len(ids) and ids[i].isdigit():
                return int(ids[i])
        return i

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu)
            self.mx = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
            self._how = "nvml"
            self._thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self._thread.start()
            return
        except Exception:
            self._how = None
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._how = "nvidia-smi"
            self._thread = threading.Thread(target=self._read_smi, daemon=True)
            self._thread.start()
        except OSError:
            self._proc = None

    def _poll_nvml(self):
        n = self._nvml
        get_reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self._stop.is_set():
            try:
                self.sm.append(float(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM)))
                self.power.append(n.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
                if get_reasons is not None:
                    mask = int(get_reasons(self._h))
                    for bit, name in self.REASONS:
                        if mask & bit:
                            self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.01)

    def _read_smi(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.strip().split(",")]
            if len(parts) < 8:
                continue
            try:
                self.sm.append(float(parts[0]))
                self.mx = float(parts[1])
                self.power.append(float(parts[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                               parts[4:8]):
                if v.lower().startswith("active"):
                    self.reasons.add(name)

    def stop(self) -> dict:
        self._stop.set()
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if self._how == "nvml":
            try:
                self._nvml.nvmlShutdown()
            except Exception:
                pass
        if self._how is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML binding and no nvidia-smi"]}
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.mx,
                "reasons": sorted(self.reasons), "samples": len(self.sm),
                "power_w": statistics.median(self.power) if self.power else None, "source": self._how}


def make_inputs(cfg, rank, dev, ring=4):
    """A ring of distinct synthetic steps in pinned host memory (tokens, per-layer top-k KV indices) + device copies."""
    import torch
    B, L = cfg.batch, cfg.n_layers
    g = torch.Generator().manual_seed(1234 + rank)
    host_tokens = [torch.randint(0, cfg.vocab, (B,), generator=g).pin_memory() for _ in range(ring)]
    host_idx = [[torch.stack([torch.randperm(cfg.ctx + 1, generator=g)[:cfg.topk_kv] for _ in range(B)])
                 .to(torch.int32).pin_memory() for _ in range(L)] for _ in range(ring)]
    return host_tokens, host_idx, [t.to(dev) for t in host_tokens], [[t.to(dev) for t in per] for per in host_idx]


class Harness:
    def __init__(self, world, dev):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.world, self.dev = torch, dist, world, dev

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


def time_product(hx, model, inputs, steps, warmup, repeats, count_launches=False):
    """Device-timed decode steps, inputs resident on the device. Step i+1's KV transfers are queued on the side
    stream as soon as step i has been launched (its indices are inputs, not model outputs). The compute stream waits
    for every queued transfer before the closing event, so each timed region holds `steps` steps of compute and
    `steps` steps of transfers. Returns (list of ms per region, launches in the last region, rows fetched per step)."""
    torch = hx.torch
    from umdk_b200 import _native
    _, _, dev_tokens, dev_idx = inputs
    ring = len(dev_tokens)
    L = model.cfg.n_layers

    def wait_prefetch():
        if model.kvm is not None:
            for l in range(L):
                model.kvm.wait(l)

    k = 0
    hx.barrier()   # the ranks built their models at their own pace: meet before the first step
    for _ in range(warmup):
        model.step(dev_tokens[k % ring], dev_idx[k % ring])
        model.prefetch(dev_idx[(k + 1) % ring], after_compute=False)
        k += 1
    torch.cuda.synchronize()
    model.check()
    out, launches, rows = [], 0, 0
    for _ in range(repeats):
        rows0 = model.kvm.rows_fetched() if (model.kvm is not None and model.rows_mode) else 0
        hx.barrier()
        l0 = _native.LAUNCH_COUNT
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            model.step(dev_tokens[k % ring], dev_idx[k % ring])
            model.prefetch(dev_idx[(k + 1) % ring], after_compute=False)
            k += 1
        wait_prefetch()
        e1.record()
        hx.barrier()
        launches = _native.LAUNCH_COUNT - l0
        if model.kvm is not None and model.rows_mode:
            rows = (model.kvm.rows_fetched() - rows0) / steps
        out.append(hx.max_over_ranks(e0.elapsed_time(e1)))
        model.check()
    wait_prefetch()
    torch.cuda.synchronize()
    model._prefetched = False
    return out, launches, rows


def time_product_e2e(hx, model, inputs, steps, warmup):
    """End to end through the public step API: every step copies, from pinned host memory, its own tokens and the
    NEXT step's KV indices (double-buffered; they feed the transfers that overlap this step), runs step(), and reads
    the sampled tokens back on the host. Returns (ms for `steps` steps, h2d bytes per step, d2h bytes per step)."""
    torch = hx.torch
    cfg = model.cfg
    B, L = cfg.batch, cfg.n_layers
    host_tokens, host_idx, _, _ = inputs
    ring = len(host_tokens)
    dev = hx.dev
    in_tokens = torch.empty(B, dtype=torch.int64, device=dev)
    in_idx = [[torch.empty(B, cfg.topk_kv, dtype=torch.int32, device=dev) for _ in range(L)] for _ in range(2)]
    host_out = torch.empty(B, dtype=torch.int64).pin_memory()
    side = model.kvm.side_stream() if model.kvm is not None else torch.cuda.current_stream()

    def stage_indices(i: int):
        buf = in_idx[i % 2]
        with torch.cuda.stream(side):   # the indices travel on the stream that consumes them
            for l in range(L):
                buf[l].copy_(host_idx[i % ring][l], non_blocking=True)
        if model.kvm is None:
            torch.cuda.current_stream().wait_stream(side)
        model.prefetch(buf, after_compute=False)

    def e2e_step(i: int):
        in_tokens.copy_(host_tokens[i % ring], non_blocking=True)
        nxt = model.step(in_tokens, in_idx[i % 2])
        stage_indices(i + 1)
        host_out.copy_(nxt, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return int(host_out[0])

    def wait_prefetch():
        if model.kvm is not None:
            for l in range(L):
                model.kvm.wait(l)

    stage_indices(0)
    for i in range(warmup):
        e2e_step(i)
    hx.barrier()
    t0 = time.perf_counter()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for i in range(steps):
        e2e_step(warmup + i)
    wait_prefetch()
    c1.record()
    hx.barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    ms = hx.max_over_ranks(max(c0.elapsed_time(c1), wall_ms))
    model.check()
    model._prefetched = False
    h2d = host_tokens[0].numel() * 8 + sum(t.numel() * 4 for t in host_idx[0])
    return ms, h2d, host_out.numel() * 8


def time_baseline(hx, cfg, inputs, steps, warmup, with_offload=True):
    """The PyTorch + NCCL + library-GEMM arm: device-timed and end-to-end tokens/s with the offloaded pages copied
    back every step, and device-timed with the whole cache resident. Frees its model before returning."""
    torch = hx.torch
    from baseline.decode_baseline import BaselineDecoderRank
    import copy
    host_tokens, host_idx, dev_tokens, dev_idx = inputs
    ring = len(dev_tokens)
    B, L = cfg.batch, cfg.n_layers
    bcfg = copy.copy(cfg)
    bcfg.offload = with_offload
    model = BaselineDecoderRank(bcfg, device=hx.dev)
    res = {"gemm": model.gemm_backend}

    def region(n, offload):
        model.offload = offload and with_offload
        k = 0
        for _ in range(max(2, warmup // 2) if n else 0):
            model.step(dev_tokens[k % ring], dev_idx[k % ring])
            model.prefetch()
            k += 1
        hx.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            model.step(dev_tokens[k % ring], dev_idx[k % ring])
            model.prefetch()
            k += 1
        model.wait_prefetch()
        e1.record()
        hx.barrier()
        model._queued = False
        return hx.max_over_ranks(e0.elapsed_time(e1))

    tokens = hx.world * B * steps
    if with_offload:
        ms = region(steps, True)
        res["tokens_per_s"], res["ms_per_step"] = tokens / (ms * 1e-3), ms / steps
        # end to end: pinned inputs in, sampled tokens out, every step
        in_tokens = torch.empty(B, dtype=torch.int64, device=hx.dev)
        in_idx = [torch.empty(B, cfg.topk_kv, dtype=torch.int32, device=hx.dev) for _ in range(L)]
        host_out = torch.empty(B, dtype=torch.int64).pin_memory()

        def e2e_step(i):
            in_tokens.copy_(host_tokens[i % ring], non_blocking=True)
            for l in range(L):
                in_idx[l].copy_(host_idx[i % ring][l], non_blocking=True)
            nxt = model.step(in_tokens, in_idx)
            model.prefetch()
            host_out.copy_(nxt, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        model.offload = True
        for i in range(2):
            e2e_step(i)
        hx.barrier()
        t0 = time.perf_counter()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for i in range(steps):
            e2e_step(2 + i)
        model.wait_prefetch()
        c1.record()
        hx.barrier()
        ms = hx.max_over_ranks(max(c0.elapsed_time(c1), (time.perf_counter() - t0) * 1e3))
        model._queued = False
        res["e2e_tokens_per_s"], res["e2e_ms_per_step"] = tokens / (ms * 1e-3), ms / steps
    ms = region(steps, False)
    res["compute_only_tokens_per_s"], res["compute_only_ms_per_step"] = tokens / (ms * 1e-3), ms / steps
    res["steps"] = steps
    model.close()
    del model
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return res


def ep_sub_metrics(rank, world, iters=10, warmup=3):
    """Configs 2 and 3 of the benchmark set (EP normal-mode dispatch / combine at 4096 tokens per rank, low-latency
    fused MoE layer at 128 tokens per rank), product and NCCL baseline, as bench/ep_bench.py measures them."""
    import types
    from bench import ep_bench
    a = types.SimpleNamespace(tokens=4096, ll_tokens=128, ll_experts=256, iters=iters, warmup=warmup, brief=True)
    recs = ep_bench.bench_normal(rank, world, a, quiet=True) + ep_bench.bench_ll(rank, world, a, quiet=True)
    out = {}
    for r in recs:
        key = None
        if r.get("config") == "ep_normal" and r.get("op", "").startswith("dispatch"):
            key = "ep_normal_dispatch"
        elif r.get("config") == "ep_normal" and r.get("op", "").startswith("combine"):
            key = "ep_normal_combine"
        elif r.get("config") == "ep_ll_moe" and ("tile-major weights (ExpertWeights.to_tiled)" in r.get("op", "")
                                                   or r.get("impl") == "nccl_grouped_gemm_baseline"):
            key = "ep_ll_layer"
        elif r.get("config") == "ep_normal" and r.get("op", "").startswith("bare"):
            key = "ep_normal_" + ("combine" if "combine" in r["op"] else "dispatch")
        if key is None:
            continue
        d = out.setdefault(key, {})
        if r.get("impl") == "umdk_b200":
            d["us"] = round(r["us"], 1)
            for f in ("nvlink_GBps", "recv_GBps", "frac_of_nvlink_roofline", "frac_of_roofline"):
                if r.get(f) is not None:
                    d[f] = round(r[f], 3)
        elif r.get("op", "").startswith("bare"):
            d["bare_all_to_all_us"] = round(r["us"], 1)
        else:
            d["baseline_us"] = round(r["us"], 1)
            if r.get("gemm"):
                d["baseline_gemm"] = r["gemm"]
    for d in out.values():
        if "us" in d and "baseline_us" in d:
            d["speedup_vs_baseline"] = round(d["baseline_us"] / d["us"], 2)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=3, help="timed regions of --steps steps each (median reported)")
    ap.add_argument("--impl", default="umdk", choices=["umdk", "baseline", "reference"])
    ap.add_argument("--config", default="full", choices=["full", "tiny"])
    ap.add_argument("--no-offload", action="store_true", help="keep the whole KV cache on the device (not the "
                    "benchmark configuration; for kernel-only studies)")
    ap.add_argument("--kv-fetch", default="rows", choices=["rows", "pages"],
                    help="how offloaded KV returns each step: the selected token rows only (gather kernel reading "
                    "pinned host memory) or all offloaded pages (cudaMemcpyAsync)")
    ap.add_argument("--no-baseline", action="store_true", help="skip the in-process baseline arm (vs_baseline null)")
    ap.add_argument("--no-extra", action="store_true", help="skip the sub-metrics under `extra`")
    ap.add_argument("--profile-step", action="store_true",
                    help="after the warm-up run ONE step between cudaProfilerStart/Stop and exit (for a launch list: "
                    "ncu --profile-from-start off --metrics gpu__time_duration.sum ...); prints no benchmark line")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.warmup < 3:
        args.warmup = 3

    import gc
    import torch
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from umdk_b200.models.dsv3_decoder import DecoderConfig, DecoderRank, build_weights

    from umdk_b200.utils.affinity import bind_to_gpu
    cpus = bind_to_gpu(local_rank)   # pinned pools land on the GPU's NUMA node
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus or world == 1, f"launched with WORLD_SIZE={world} but --gpus {args.gpus}"
    hx = Harness(world, dev)

    cfg = DecoderConfig() if args.config == "full" else DecoderConfig.tiny()
    cfg.offload = not args.no_offload
    cfg.kv_fetch = args.kv_fetch
    B = cfg.batch
    inputs = make_inputs(cfg, rank, dev)
    model_name = "deepseek-v3-shaped 4-layer MoE decoder" if args.config == "full" else "tiny"
    common_cfg = {"model": model_name, "global_batch": world * B, "seq_len": cfg.ctx,
                  "parallelism": f"ep{world}+dp{world}", "experts": cfg.n_experts, "top_k": cfg.top_k,
                  "moe_ffn": cfg.moe_ffn, "hidden": cfg.hidden, "kv_topk": cfg.topk_kv, "kv_page": 64,
                  "l2": "per-step working set (expert weights + KV) is far larger than the 126 MB L2"}

    # ---- the PyTorch + NCCL + library-GEMM arm (first, then freed) ----
    base = None
    if args.impl == "baseline" or not args.no_baseline:
        sampler = ClockSampler(local_rank) if args.impl == "baseline" else None
        if sampler:
            sampler.start()
        base = time_baseline(hx, cfg, inputs, args.steps if args.impl == "baseline" else min(args.steps, 10),
                             args.warmup, with_offload=cfg.offload)
        if args.impl == "baseline":
            clocks = sampler.stop()
            if rank == 0:
                v = base.get("tokens_per_s", base["compute_only_tokens_per_s"])
                print(json.dumps({
                    "metric": "moe_decode_tokens_per_sec_per_box", "value": v, "unit": "tokens/s", "n_gpus": world,
                    "steps": args.steps, "warmup": args.warmup,
                    "ms_per_step": base.get("ms_per_step", base["compute_only_ms_per_step"]),
                    "higher_is_better": True, "scaling": "weak", "vs_baseline": 1.0,
                    "dtype": "bf16 activations/KV, expert GEMMs: " + base["gemm"],
                    "data": "synthetic (random-init weights, random KV cache, random top-2048 indices)",
                    "impl": "nccl_baseline (PyTorch + NCCL + library GEMMs; none of this package's kernels)",
                    "config": dict(common_cfg, kv_offload="every offloaded page copied back each step with "
                                   "cudaMemcpyAsync on a side stream" if cfg.offload else "off"),
                    "clocks": clocks, "e2e": {"value": base.get("e2e_tokens_per_s"), "unit": "tokens/s"},
                    "gpu_launches": 0, "extra": base}))
            if world > 1:
                dist.destroy_process_group()
            return 0

    weights = build_weights(cfg, dev, rank, world)
    model = DecoderRank(cfg, device=dev, weights=weights)
    L = cfg.n_layers

    if args.profile_step:
        _, _, dev_tokens, dev_idx = inputs
        for i in range(args.warmup):
            model.step(dev_tokens[i % 4], dev_idx[i % 4])
            model.prefetch(dev_idx[(i + 1) % 4], after_compute=False)
        torch.cuda.synchronize()
        model.check()
        torch.cuda.profiler.start()
        model.step(dev_tokens[0], dev_idx[args.warmup % 4])
        if model.kvm is not None:
            for l in range(L):
                model.kvm.wait(l)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        model.close()
        return 0

    sampler = ClockSampler(local_rank)
    sampler.start()
    regions, launches, rows_per_step = time_product(hx, model, inputs, args.steps, args.warmup, max(1, args.repeats))
    clocks = sampler.stop()
    ms = statistics.median(regions)
    e2e_ms, h2d_bytes, d2h_bytes = time_product_e2e(hx, model, inputs, args.steps, args.warmup)
    kv_stats = model.kvm.stats() if model.kvm is not None else {"bytes_h2d": 0, "copies": 0}
    rows_mode, n_staging = model.rows_mode, model.n_staging
    model.close()
    del model
    gc.collect()
    torch.cuda.empty_cache()

    tokens = world * B * args.steps
    value = tokens / (ms * 1e-3)
    e2e_value = tokens / (e2e_ms * 1e-3)
    if not cfg.offload:
        kv_bytes_step, kv_how = 0, "off"
    elif rows_mode:
        kv_bytes_step = int(rows_per_step * 576 * 2)
        kv_how = ("half of each sequence's pages in pinned host memory (moved out with cudaMemcpyAsync on a side "
                  "stream); every step a gather kernel on the side stream reads the token rows that the step's "
                  "top-2048 indices select straight from the pinned pool into a device landing area")
    else:
        kv_bytes_step = cfg.n_layers * n_staging * 64 * 576 * 2
        kv_how = ("half of each sequence's pages in pinned host memory, all of them prefetched every step with "
                  "cudaMemcpyAsync on a side stream")

    # ---- the other named sub-metrics ----
    extra = {}
    if base is not None:
        extra["baseline"] = base
    if not args.no_extra:
        import copy
        n_extra = min(args.steps, 10)
        for name, off, fetch in (("pages_mode", True, "pages"), ("compute_only", False, "rows")):
            if (off, fetch) == (cfg.offload, cfg.kv_fetch) or (not off and not cfg.offload):
                continue
            c2 = copy.copy(cfg)
            c2.offload, c2.kv_fetch = off, fetch
            m2 = DecoderRank(c2, device=dev, weights=weights)
            r2, _, _ = time_product(hx, m2, inputs, n_extra, 3, 1)
            extra[name] = {"tokens_per_s": world * B * n_extra / (r2[0] * 1e-3), "ms_per_step": r2[0] / n_extra,
                           "steps": n_extra}
            m2.close()
            del m2
            gc.collect()
            torch.cuda.empty_cache()
        if base is not None and "compute_only" in extra:
            extra["compute_only"]["vs_baseline"] = extra["compute_only"]["tokens_per_s"] / \
                base["compute_only_tokens_per_s"]
        if base is not None and "pages_mode" in extra and "tokens_per_s" in base:
            extra["pages_mode"]["vs_baseline"] = extra["pages_mode"]["tokens_per_s"] / base["tokens_per_s"]
    del weights
    gc.collect()
    torch.cuda.empty_cache()
    if not args.no_extra and world > 1 and args.config == "full":
        try:
            extra.update(ep_sub_metrics(rank, world))
        except Exception as e:  # noqa: BLE001 - the headline line must still be printed
            extra["ep_sub_metrics_error"] = f"{type(e).__name__}: {str(e)[:200]}"

    base_key = "tokens_per_s" if cfg.offload else "compute_only_tokens_per_s"
    vs_baseline = value / base[base_key] if base is not None else None
    e2e_vs = (e2e_value / base["e2e_tokens_per_s"]) if (base is not None and "e2e_tokens_per_s" in base) else None
    if rank == 0:
        print(json.dumps({
            "metric": "moe_decode_tokens_per_sec_per_box", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": vs_baseline,
            "baseline_is": "the same decode step on PyTorch + NCCL + library GEMMs, timed in this process on this "
                           "box (the reference project has no code that runs on NVIDIA GPUs and publishes no number "
                           "for this workload)",
            "dtype": "bf16 activations/KV, fp8-e4m3 expert GEMMs",
            "data": "synthetic (random-init weights, random KV cache, random top-2048 indices)",
            "impl": "umdk_b200",
            "config": dict(common_cfg, kv_offload=kv_how, kv_fetch=cfg.kv_fetch if cfg.offload else None,
                           kv_prefetch_bytes_per_step_per_gpu=kv_bytes_step),
            "repeats": {"ms_per_step": [r / args.steps for r in regions], "min": min(regions) / args.steps,
                        "median": ms / args.steps},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes, "vs_baseline": e2e_vs},
            "gpu_launches": launches,
            "cpu_affinity": f"{len(cpus)} CPUs local to GPU {local_rank}" if cpus else "unchanged",
            "kv_copies_total": kv_stats["copies"],
            "extra": extra,
        }))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
