"""Rotary position encoding: rotate-half on query and key heads, values untouched.

Inverse frequencies in float32 as the reference computes them (fusezap/serve/models/llama.py:102-120):
`inv[j] = 1 / theta^(2j/hd)`; `linear`: `inv / factor`; `llama3`: with `wl = 2*pi/inv`, frequencies whose wavelength
exceeds `old/low` are divided by `factor`, those between `old/high` and `old/low` are blended with
`smooth = (old/wl - low) / (high - low)`. Tables `cos(p * inv[j])`, `sin(...)` of shape (max_len, hd/2) in float32
(llama.py:122-130); the rotation itself (llama.py:524-527): `out = cat(x1*cos - x2*sin, x2*cos + x1*sin)` with
`x1 = x[..., :hd/2]`, `x2 = x[..., hd/2:]`, the row of the token's own position. The angles and the rotation are computed in
32-bit in both dtypes; the result is rounded once to the cache's dtype.
"""
from __future__ import annotations
import math

import numpy as np
import torch

from .base import LayerCache, PositionEncoding, register_position


def inverse_frequencies(head_dim: int, theta: float, kind: str = "default", factor: float = 1.0,
                        low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                        original_max_position_embeddings: int = 0) -> np.ndarray:
    d = head_dim
    inv = (1.0 / (np.float32(theta) ** (np.arange(0, d, 2, dtype=np.int64).astype(np.float32) / np.float32(d)))).astype(np.float32)
    if kind == "linear":
        inv = (inv / np.float32(factor)).astype(np.float32)
    elif kind == "llama3":
        old, lo, hi = original_max_position_embeddings, low_freq_factor, high_freq_factor
        wl = 2 * math.pi / inv
        smooth = (old / wl - lo) / (hi - lo)
        out = np.where(wl > old / lo, inv / factor, inv)
        mid = (wl <= old / lo) & (wl >= old / hi)
        inv = np.where(mid, (1 - smooth) * out / factor + smooth * out, out).astype(np.float32)
    elif kind != "default":
        raise NotImplementedError(f"rope kind {kind!r}")
    return inv


@register_position("rope")
class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, kind: str = "default", factor: float = 1.0,
                 low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                 original_max_position_embeddings: int = 0):
        if head_dim % 2:
            raise ValueError(f"rope needs an even head_dim, got {head_dim}")
        self.head_dim = head_dim
        self.inv_freq = inverse_frequencies(head_dim, theta, kind, factor, low_freq_factor, high_freq_factor,
                                            original_max_position_embeddings)
        self.cos: torch.Tensor | None = None
        self.sin: torch.Tensor | None = None

    def prepare(self, max_len: int, device: torch.device) -> None:
        fr = np.arange(max_len, dtype=np.float32)[:, None] * self.inv_freq[None, :]
        self.cos = torch.from_numpy(np.cos(fr).astype(np.float32)).to(device)
        self.sin = torch.from_numpy(np.sin(fr).astype(np.float32)).to(device)

    def weight_tensors(self) -> list:
        return []       # a step gathers one row of the tables per token; they are not streamed like weights

    def rotate_and_store(self, ctx, qkv: torch.Tensor, q_out: torch.Tensor, cache: LayerCache,
                         num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        if head_dim != self.head_dim:
            raise ValueError(f"rope was built for head_dim {self.head_dim}, the mixer has {head_dim}")
        ctx.ops.rope_kv_write(qkv, self.cos, self.sin, ctx.meta, cache, q_out, num_heads, num_kv_heads, head_dim)

    def project_rotate_store(self, ctx, h, w, bias, q_out, cache, num_heads, num_kv_heads, head_dim) -> bool:
        if head_dim != self.head_dim:
            raise ValueError(f"rope was built for head_dim {self.head_dim}, the mixer has {head_dim}")
        fused = getattr(ctx.ops, "linear_rope_kv_write", None)      # an optional entry of the kernel table
        return bool(fused is not None and fused(h, w, bias, self.cos, self.sin, ctx.meta, cache, q_out, num_heads,
                                                num_kv_heads, head_dim))
