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

Rank 0 prints ONE JSON line. `value` is device-timed (CUDA events, max over ranks) with inputs resident on the
device; `e2e.value` goes through the public `DecoderRank.step` API with the step's inputs copied from pinned host
memory and the sampled tokens read back on the host every step.
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="umdk", choices=["umdk", "reference"])
    ap.add_argument("--config", default="full", choices=["full", "tiny"])
    ap.add_argument("--no-offload", action="store_true", help="keep the whole KV cache on the device (not the "
                    "benchmark configuration; for kernel-only studies)")
    ap.add_argument("--kv-fetch", default="rows", choices=["rows", "pages"],
                    help="how offloaded KV returns each step: the selected token rows only (gather kernel reading "
                    "pinned host memory) or all offloaded pages (cudaMemcpyAsync)")
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

    import torch
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from umdk_b200 import _native
    from umdk_b200.models.dsv3_decoder import DecoderConfig, DecoderRank

    from umdk_b200.utils.affinity import bind_to_gpu
    cpus = bind_to_gpu(local_rank)   # pinned pools land on the GPU's NUMA node
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus or world == 1, f"launched with WORLD_SIZE={world} but --gpus {args.gpus}"

    cfg = DecoderConfig() if args.config == "full" else DecoderConfig.tiny()
    cfg.offload = not args.no_offload
    cfg.kv_fetch = args.kv_fetch
    model = DecoderRank(cfg, device=dev)
    B, L = cfg.batch, cfg.n_layers

    # synthetic inputs of the named shape: a ring of distinct steps in pinned host memory
    ring = 4
    g = torch.Generator().manual_seed(1234 + rank)
    host_tokens = [torch.randint(0, cfg.vocab, (B,), generator=g).pin_memory() for _ in range(ring)]
    host_idx = [[torch.stack([torch.randperm(cfg.ctx + 1, generator=g)[:cfg.topk_kv] for _ in range(B)])
                 .to(torch.int32).pin_memory() for _ in range(L)] for _ in range(ring)]
    dev_tokens = [t.to(dev) for t in host_tokens]
    dev_idx = [[t.to(dev) for t in per] for per in host_idx]
    in_tokens = torch.empty(B, dtype=torch.int64, device=dev)
    in_idx = [[torch.empty(B, cfg.topk_kv, dtype=torch.int32, device=dev) for _ in range(L)] for _ in range(2)]
    host_out = torch.empty(B, dtype=torch.int64).pin_memory()
    h2d_bytes = host_tokens[0].numel() * 8 + sum(t.numel() * 4 for t in host_idx[0])
    d2h_bytes = host_out.numel() * 8

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def wait_prefetch():
        if model.kvm is not None:
            for l in range(L):
                model.kvm.wait(l)

    # ---- device-timed: inputs resident on the device ----
    # Step i+1's KV transfers are queued on the side stream as soon as step i has been launched (its indices are
    # inputs, not model outputs). The compute stream waits for every queued transfer before the closing event, so
    # the timed region holds K steps of compute and K steps of transfers.
    for i in range(args.warmup):
        model.step(dev_tokens[i % ring], dev_idx[i % ring])
        model.prefetch(dev_idx[(i + 1) % ring], after_compute=False)
    torch.cuda.synchronize()
    model.check()
    if args.profile_step:
        torch.cuda.profiler.start()
        model.step(dev_tokens[0], dev_idx[args.warmup % ring])
        wait_prefetch()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        model.close()
        return 0
    rows0 = model.kvm.rows_fetched() if (model.kvm is not None and model.rows_mode) else 0
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    launches0 = _native.LAUNCH_COUNT
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        k = args.warmup + i
        model.step(dev_tokens[k % ring], dev_idx[k % ring])
        model.prefetch(dev_idx[(k + 1) % ring], after_compute=False)
    wait_prefetch()
    e1.record()
    barrier()
    rows_per_step = ((model.kvm.rows_fetched() - rows0) / args.steps
                     if (model.kvm is not None and model.rows_mode) else 0)
    launches = _native.LAUNCH_COUNT - launches0
    ms = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop()
    model.check()

    # ---- end to end through the public step API: pinned host inputs in, sampled tokens out, every step ----
    # Every step copies, from pinned host memory, its own tokens and the NEXT step's KV indices (double-buffered;
    # they feed the transfers that overlap this step), runs the public step(), and reads the sampled tokens back.
    side = model.kvm.side_stream() if model.kvm is not None else torch.cuda.current_stream()

    def stage_indices(i: int):
        buf = in_idx[i % 2]
        with torch.cuda.stream(side):   # the indices travel on the stream that consumes them
            for l in range(L):
                buf[l].copy_(host_idx[i % ring][l], non_blocking=True)
        model.prefetch(buf, after_compute=False)

    def e2e_step(i: int):
        in_tokens.copy_(host_tokens[i % ring], non_blocking=True)
        nxt = model.step(in_tokens, in_idx[i % 2])
        stage_indices(i + 1)
        host_out.copy_(nxt, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return int(host_out[0])

    wait_prefetch()          # the transfer queued by the last device-timed step used other index buffers
    torch.cuda.synchronize()
    model._prefetched = False
    stage_indices(0)
    for i in range(args.warmup):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for i in range(args.steps):
        e2e_step(args.warmup + i)
    wait_prefetch()
    c1.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(max(c0.elapsed_time(c1), wall_ms))
    model.check()
    kv_stats = model.kvm.stats() if model.kvm is not None else {"bytes_h2d": 0, "copies": 0}

    tokens = world * B * args.steps
    value = tokens / (ms * 1e-3)
    e2e_value = tokens / (e2e_ms * 1e-3)
    if not cfg.offload:
        kv_bytes_step, kv_how = 0, "off"
    elif model.rows_mode:
        kv_bytes_step = int(rows_per_step * 576 * 2)
        kv_how = ("half of each sequence's pages in pinned host memory (moved out with cudaMemcpyAsync on a side "
                  "stream); every step a gather kernel on the side stream reads the token rows that the step's "
                  "top-2048 indices select straight from the pinned pool into a device landing area")
    else:
        kv_bytes_step = cfg.n_layers * model.n_staging * 64 * 576 * 2
        kv_how = ("half of each sequence's pages in pinned host memory, all of them prefetched every step with "
                  "cudaMemcpyAsync on a side stream")
    if rank == 0:
        print(json.dumps({
            "metric": "moe_decode_tokens_per_sec_per_box", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations/KV, fp8-e4m3 expert GEMMs",
            "data": "synthetic (random-init weights, random KV cache, random top-2048 indices)",
            "impl": "umdk_b200",
            "config": {"model": "deepseek-v3-shaped 4-layer MoE decoder" if args.config == "full" else "tiny",
                       "global_batch": world * B, "seq_len": cfg.ctx, "parallelism": f"ep{world}+dp{world}",
                       "experts": cfg.n_experts, "top_k": cfg.top_k, "moe_ffn": cfg.moe_ffn, "hidden": cfg.hidden,
                       "kv_topk": cfg.topk_kv, "kv_page": 64, "kv_offload": kv_how, "kv_fetch": cfg.kv_fetch if cfg.offload else None,
                       "kv_prefetch_bytes_per_step_per_gpu": kv_bytes_step,
                       "l2": "per-step working set (expert weights + KV) is far larger than the 126 MB L2"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
            "gpu_launches": launches,
            "cpu_affinity": f"{len(cpus)} CPUs local to GPU {local_rank}" if cpus else "unchanged",
            "kv_copies_total": kv_stats["copies"],
        }))
    model.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
