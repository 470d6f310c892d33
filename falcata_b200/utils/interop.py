"""Zero-copy views between raw device pointers owned by the native core and torch tensors."""
from __future__ import annotations

from typing import Sequence

import numpy as np


class _CudaArrayView:
    """Minimal ``__cuda_array_interface__`` carrier for memory owned by the native core."""

    def __init__(self, ptr: int, shape: Sequence[int], typestr: str) -> None:
        self.__cuda_array_interface__ = {"shape": tuple(int(s) for s in shape), "typestr": typestr, "data": (int(ptr), False), "version": 2, "strides": None}


def tensor_from_ptr(ptr: int, shape: Sequence[int], dtype):
    """torch CUDA tensor aliasing ``ptr`` (no copy, no ownership)."""
    import torch

    typestr = {torch.float32: "<f4", torch.float64: "<f8", torch.int32: "<i4", torch.uint8: "|u1", torch.int64: "<i8"}[dtype]
    return torch.as_tensor(_CudaArrayView(ptr, shape, typestr), device="cuda")
