"""Grouped-query attention over the paged cache.

In the order the reference runs it (fusezap/serve/models/llama.py:570-594, 724-736): one product with the rows
[q; k; v] stacked at load (llama.py:293-295, 325), bias added when the checkpoint has q/k/v biases (all three or none);
rotation of q and k by the token's position and the write of k, v into the request's pages; then for the token at
position p the keys 0..p of its own request (the last `window` of them if the layer has a window: positions
p-window+1..p, fusezap/serve/models/swa.py:74-77), query head h reading kv head h // (Hq/Hkv), scores `(q.k) * scale`,
softmax, values; then the output product, whose result is the residual term. Scores, softmax and the value sum are in
32-bit in both dtypes.
"""
from __future__ import annotations
import torch

from ..cache import KVNeed
from ..weights import ParamSpec
from .base import LayerCache, Mixer, register_mixer


@register_mixer("gqa_attention")
class GQAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 window: int = 0, position: str | None = "rope",
                 names: tuple[str, str, str, str] = ("q_proj", "k_proj", "v_proj", "o_proj")):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
        self.D, self.Hq, self.Hkv, self.hd = hidden_size, num_heads, num_kv_heads, head_dim
        self.scale, self.window, self.position, self.names = float(scale), int(window), position, tuple(names)
        self.wqkv = self.bqkv = self.wo = self.bo = None

    def tensors(self) -> dict[str, ParamSpec]:
        q, k, v, o = self.names
        D, Hq, Hkv, hd = self.D, self.Hq, self.Hkv, self.hd
        return {
            f"{q}.weight": ParamSpec((Hq * hd, D)), f"{k}.weight": ParamSpec((Hkv * hd, D)),
            f"{v}.weight": ParamSpec((Hkv * hd, D)), f"{o}.weight": ParamSpec((D, Hq * hd)),
            f"{q}.bias": ParamSpec((Hq * hd,), role="vector", group="qkv_bias"),
            f"{k}.bias": ParamSpec((Hkv * hd,), role="vector", group="qkv_bias"),
            f"{v}.bias": ParamSpec((Hkv * hd,), role="vector", group="qkv_bias"),
            f"{o}.bias": ParamSpec((D,), role="vector", group="o_bias"),
        }

    def bind(self, tensors, ops) -> None:
        q, k, v, o = self.names
        self.wqkv = torch.cat([tensors[f"{q}.weight"], tensors[f"{k}.weight"], tensors[f"{v}.weight"]], 0).contiguous()
        if f"{q}.bias" in tensors:
            self.bqkv = torch.cat([tensors[f"{n}.bias"].float() for n in (q, k, v)], 0).contiguous()
        self.wo = tensors[f"{o}.weight"]
        self.bo = tensors[f"{o}.bias"].float() if f"{o}.bias" in tensors else None
        ops.check_attention(self.Hq, self.Hkv, self.hd)

    def cache_need(self) -> KVNeed:
        return KVNeed(self.Hkv, self.hd, self.window)

    def position_name(self) -> str | None:
        return self.position

    def step_needs(self) -> tuple[str, ...]:
        return ("attention",)

    def forward(self, ctx, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        n, ops, ws = h.shape[0], ctx.ops, ctx.ws
        Hq, Hkv, hd = self.Hq, self.Hkv, self.hd
        q = ws.get("q", (n, Hq * hd), ops.dtype)
        position = ctx.positions[self.position]
        if not position.project_rotate_store(ctx, h, self.wqkv, self.bqkv, q, cache, Hq, Hkv, hd):
            qkv = ws.get("qkv", (n, (Hq + 2 * Hkv) * hd), torch.float32)
            ops.linear(h, self.wqkv, self.bqkv, qkv)
            position.rotate_and_store(ctx, qkv, q, cache, Hq, Hkv, hd)
        o = ws.get("attn_out", (n, Hq * hd), ops.dtype)
        ops.paged_attention(q, cache, ctx.meta, o, Hq, Hkv, hd, self.scale, self.window)
        delta = ws.get("delta", (n, self.D), torch.float32)
        ops.linear(o, self.wo, self.bo, delta)
        return delta
