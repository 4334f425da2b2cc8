"""The CUDA kernels (csrc/), their build and the kernel table the parts call."""
from __future__ import annotations
from .interface import Ops

_tables: dict = {}


def cuda_ops(dtype: str, device="cuda:0"):
    """The kernel table for `dtype` on `device` (built once per pair). Raises if there is no GPU or no compiler."""
    import torch
    from .table import CudaOps
    key = (str(dtype), str(torch.device(device)))
    if key not in _tables:
        _tables[key] = CudaOps(dtype, device)
    return _tables[key]


__all__ = ["Ops", "cuda_ops"]
