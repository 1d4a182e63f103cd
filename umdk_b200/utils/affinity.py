"""CPU / NUMA placement of a rank process next to its GPU.

Pinned host memory (the KV offload pool, staging buffers) is allocated on the NUMA node of the thread that allocates
it; a rank whose GPU hangs off the other socket would pull every PCIe read across the inter-socket link. Binding the
process to the CPUs NVML reports as local to the GPU - before anything is allocated - keeps the pool on the right
node. Read-only use of NVML; nothing about the GPU is changed.
"""
from __future__ import annotations

import os
from typing import List, Optional


def gpu_local_cpus(device_index: int) -> Optional[List[int]]:
    """CPUs that NVML lists as local to the GPU, or None if NVML is not usable."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = device_index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if device_index < len(ids) and ids[device_index].isdigit():
                    phys = int(ids[device_index])
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            ncpu = os.cpu_count() or 64
            words = pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
            cpus = [w * 64 + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1]
            return cpus or None
        finally:
            pynvml.nvmlShutdown()
    except Exception:
        return None


def bind_to_gpu(device_index: int) -> Optional[List[int]]:
    """Restricts this process to the CPUs local to the GPU (intersected with what it may already use).
    Returns the CPU list it ended up with, or None if nothing was changed."""
    cpus = gpu_local_cpus(device_index)
    if not cpus:
        return None
    try:
        allowed = os.sched_getaffinity(0)
        target = sorted(set(cpus) & set(allowed))
        if not target:
            return None
        os.sched_setaffinity(0, target)
        return target
    except (AttributeError, OSError):
        return None
