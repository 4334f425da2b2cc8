"""RMSNorm with the residual add folded in.

`x <- x + delta` (the pending term of the previous sublayer), then `h = w * (x / sqrt(mean(x^2) + eps))`
(fusezap/serve/models/llama.py:500-503, 508-523: `mean = sum * (1/D)`, the fused kernel also writes the residual
stream). The residual stream x is float32 in both dtypes; the sum of squares, the scale and the weight product are
computed in 32-bit and h is rounded once to the activation dtype.
"""
from __future__ import annotations
import torch

from ..weights import ParamSpec
from .base import Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, size: int, eps: float):
        self.size, self.eps = size, float(eps)
        self.weight: torch.Tensor | None = None

    def tensors(self) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), role="vector", init="ones")}

    def bind(self, tensors, ops) -> None:
        self.weight = tensors["weight"]

    def forward(self, ctx, x, delta, rows=None, n_rows=None):
        n = x.shape[0] if rows is None else (n_rows if n_rows is not None else rows.shape[0])
        h = ctx.ws.get("norm_h" if rows is None else "norm_h_rows", (n, self.size), ctx.ops.dtype)
        ctx.ops.add_rmsnorm(x, delta, self.weight, self.eps, h, rows)
        return h
