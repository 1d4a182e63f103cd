"""Dense bf16 GEMM on tcgen05 / TMEM: C = A @ B^T with A [M, K], B [N, K] (both K-major), C [M, N], fp32 accumulation.

Two kernels: one CTA per 128 x 256 tile (csrc/cam/gemm_bf16.cu, any shape with N a multiple of 8) and one CTA PAIR per
256 x 256 tile (csrc/cam/gemm_bf16_2sm.cu, M and N multiples of 256, K a multiple of 64). ``impl="auto"`` picks the
pair kernel where it applies. The tensor-parallel fused ops build on the same main loop.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from .ep import check_status


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, impl: str = "auto",
              status: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
    assert a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1]
    assert a.stride(1) == 1 and b.stride(1) == 1
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    assert out.stride(1) == 1
    own_status = status is None
    if own_status:
        status = torch.zeros(4, dtype=torch.int32, device=a.device)
    pair_ok = M % 256 == 0 and N % 256 == 0 and K % 64 == 0
    if impl == "auto":
        impl = "2sm" if pair_ok else "1sm"
    lib = _native.cam()
    fn = lib.umdk_gemm_bf16_2sm if impl == "2sm" else lib.umdk_gemm_bf16
    rc = fn(_native.ptr(a), _native.ptr(b), _native.ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0),
            _native.ptr(status), _native.stream_ptr(), max_ctas)
    if rc != 0:
        raise RuntimeError(f"gemm_bf16({impl}) failed: {rc}")
    if own_status:
        check_status(status, f"gemm_bf16({impl})")
    return out
