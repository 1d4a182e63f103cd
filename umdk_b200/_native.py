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


def cam() -> ctypes.CDLL:
    """CUDA kernels + symmetric-heap runtime (sm_100a)."""
    return _load("umdk_cam", "umdk_cam")


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
