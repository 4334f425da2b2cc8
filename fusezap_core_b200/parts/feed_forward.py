"""SwiGLU feed-forward: `down(silu(gate(h)) * up(h))`.

One product with the rows [gate; up] stacked at load (fusezap/serve/models/llama.py:327, 746-749), `silu(g) = g / (1 +
exp(-g))` in 32-bit (fusezap/serve/cuda.py:284-303), then the down product (llama.py:752), whose result is the residual
term. Optional biases are taken when the checkpoint has them (gate and up together; down). Where the kernel table has
a fused kernel, the gate/up product and the activation run as one launch and the (N, 2 I) intermediate never exists.
"""
from __future__ import annotations
import torch

from ..weights import ParamSpec
from .base import FeedForward, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int,
                 names: tuple[str, str, str] = ("gate_proj", "up_proj", "down_proj")):
        self.D, self.I, self.names = hidden_size, intermediate_size, tuple(names)
        self.wgu = self.bgu = self.wd = self.bd = self.packed = None

    def tensors(self) -> dict[str, ParamSpec]:
        g, u, d = self.names
        return {
            f"{g}.weight": ParamSpec((self.I, self.D)), f"{u}.weight": ParamSpec((self.I, self.D)),
            f"{d}.weight": ParamSpec((self.D, self.I)),
            f"{g}.bias": ParamSpec((self.I,), role="vector", group="gate_up_bias"),
            f"{u}.bias": ParamSpec((self.I,), role="vector", group="gate_up_bias"),
            f"{d}.bias": ParamSpec((self.D,), role="vector", group="down_bias"),
        }

    def bind(self, tensors, ops) -> None:
        g, u, d = self.names
        # the kernel table may want gate and up in a layout of its own for a fused product + activation
        self.packed = ops.pack_gate_up(tensors[f"{g}.weight"], tensors[f"{u}.weight"], tensors.get(f"{g}.bias"),
                                       tensors.get(f"{u}.bias"))
        if self.packed is None:
            self.wgu = torch.cat([tensors[f"{g}.weight"], tensors[f"{u}.weight"]], 0).contiguous()
            if f"{g}.bias" in tensors:
                self.bgu = torch.cat([tensors[f"{g}.bias"].float(), tensors[f"{u}.bias"].float()], 0).contiguous()
        self.wd = tensors[f"{d}.weight"]
        self.bd = tensors[f"{d}.bias"].float() if f"{d}.bias" in tensors else None

    def forward(self, ctx, h: torch.Tensor) -> torch.Tensor:
        n, ops, ws = h.shape[0], ctx.ops, ctx.ws
        a = ws.get("act", (n, self.I), ops.dtype)
        if self.packed is not None:
            ops.linear_swiglu(h, self.packed, a)
        else:
            gu = ws.get("gate_up", (n, 2 * self.I), ops.dtype)
            ops.linear(h, self.wgu, self.bgu, gu)
            ops.swiglu(gu, a)
        delta = ws.get("delta", (n, self.D), torch.float32)
        ops.linear(a, self.wd, self.bd, delta)
        return delta
