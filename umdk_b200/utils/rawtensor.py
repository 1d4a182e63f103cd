"""Wrap raw device pointers (symmetric-heap regions) as torch tensors without copying."""
from __future__ import annotations

import math

import torch


class _CudaArray:
    """Minimal object exposing __cuda_array_interface__ so torch.as_tensor can adopt a raw device pointer."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


def from_ptr(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    n = math.prod(shape)
    itemsize = torch.empty((), dtype=dtype).element_size()
    raw = torch.as_tensor(_CudaArray(ptr, n * itemsize), device=device)
    return raw.view(dtype).reshape(shape)
