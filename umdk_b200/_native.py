"""ctypes loaders for the in-tree native libraries.

The CUDA library (``libumdk_cam.so``) is mandatory on a machine with a GPU: :func:`cam` raises if it is missing
instead of letting callers fall back to PyTorch silently. Host libraries (URMA, UMQ, URPC, DLock, USOCK) are plain
C++ and load everywhere.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent / "_lib"
_cache: dict[str, ctypes.CDLL] = {}


class NativeLibraryMissing(RuntimeError):
    pass


def lib_dir() -> Path:
    return _LIB_DIR


def _load(name: str, build_hint: str) -> ctypes.CDLL:
    if name in _cache:
        return _cache[name]
    path = _LIB_DIR / f"lib{name}.so"
    if not path.exists():
        if os.environ.get("UMDK_AUTO_BUILD", "1") == "1":
            from . import _build
            _build.build_all(only=build_hint.split(","))
        if not path.exists():
            raise NativeLibraryMissing(f"{path} not built; run `python -m umdk_b200._build`")
    mode = ctypes.RTLD_GLOBAL
    lib = ctypes.CDLL(str(path), mode=mode)
    _cache[name] = lib
    return lib


# Entry points of libumdk_cam.so that launch at least one hand-written kernel, with the number of kernels each
# call launches. Used to count launches for the benchmark's `gpu_launches` claim.
_KERNEL_ENTRY_POINTS = {
    "umdk_gemm_bf16": 1, "umdk_ep_layout": 1, "umdk_ep_dispatch": 1, "umdk_ep_combine": 1, "umdk_moe_gemm": 1,
    "umdk_ep_ll_dispatch": 1, "umdk_quant_fp8_1x128": 1, "umdk_sparse_mla_decode": 1, "umdk_allreduce": 1,
    "umdk_ag_gemm": 1, "umdk_gemm_rs": 1, "umdk_moe_fused": 1, "umdk_tp_gemm": 1, "umdk_gemm_bf16_2sm": 1,
    "umdk_kv_prefetch_rows": 1, "umdk_ep_notify": 1, "umdk_add_rmsnorm": 1, "umdk_qkv_post": 1, "umdk_q_rope": 1,
    "umdk_router_topk": 1, "umdk_ep_ll_combine": 1,
}
LAUNCH_COUNT = 0


class _CountingLib:
    """Proxy over the ctypes library that counts calls of kernel-launching entry points."""

    def __init__(self, lib: ctypes.CDLL):
        object.__setattr__(self, "_lib", lib)
        object.__setattr__(self, "_wrapped", {})

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        n = _KERNEL_ENTRY_POINTS.get(name)
        if n is None:
            return fn
        w = self._wrapped.get(name)
        if w is None:
            def w(*args, _fn=fn, _n=n):
                global LAUNCH_COUNT
                LAUNCH_COUNT += _n
                return _fn(*args)
            self._wrapped[name] = w
        return w


_cam_proxy = None


def cam():
    """CUDA kernels + symmetric-heap runtime (sm_100a)."""
    global _cam_proxy
    if _cam_proxy is None:
        _cam_proxy = _CountingLib(_load("umdk_cam", "umdk_cam"))
    return _cam_proxy


def urma() -> ctypes.CDLL:
    return _load("umdk_urma", "umdk_urma")


def umq() -> ctypes.CDLL:
    urma()
    return _load("umdk_umq", "umdk_urma,umdk_umq")


def urpc() -> ctypes.CDLL:
    umq()
    return _load("umdk_urpc", "umdk_urma,umdk_umq,umdk_urpc")


def dlock() -> ctypes.CDLL:
    urma()
    return _load("umdk_dlock", "umdk_urma,umdk_dlock")


def usock() -> ctypes.CDLL:
    return _load("umdk_usock", "umdk_usock")


def tool_path(name: str) -> Path:
    return _LIB_DIR / "bin" / name


def ptr(t) -> ctypes.c_void_p:
    """Device/host pointer of a torch tensor (None -> NULL)."""
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def stream_ptr() -> ctypes.c_void_p:
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
