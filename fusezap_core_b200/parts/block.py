"""Pre-norm block: `x += mixer(norm1(x)); x += ffn(norm2(x))`.

The sublayer outputs are not added at once: each norm adds the pending term of the sublayer before it, in one pass
over the row (fusezap/serve/models/llama.py:568, 600, 606: `x, h = add_norm(x, d, ln)`), and the model adds the last
one before the final norm (llama.py:608, 755).
"""
from __future__ import annotations
from ..weights import ParamSpec
from .base import Block, FeedForward, LayerCache, Mixer, Norm, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    def __init__(self, mixer: Mixer, ffn: FeedForward, make_norm,
                 names: tuple[str, str, str, str] = ("input_layernorm", "self_attn", "post_attention_layernorm", "mlp"),
                 norms: tuple = (None, None)):
        """mixer, ffn: the layer's built parts; make_norm(spec): builds a norm. `norms`: a PartSpec for the norm before
        the mixer and one for the norm before the feed-forward (None: the layer's fallback kind), so the two may be of
        different kinds."""
        self.mixer, self.ffn, self.names = mixer, ffn, tuple(names)
        self.norm1, self.norm2 = (make_norm(spec) if spec is not None else make_norm() for spec in norms)

    def children(self):
        n1, mx, n2, ff = self.names
        return ((n1, self.norm1), (mx, self.mixer), (n2, self.norm2), (ff, self.ffn))

    def tensors(self) -> dict[str, ParamSpec]:
        return {f"{prefix}.{k}": v for prefix, part in self.children() for k, v in part.tensors().items()}

    def bind(self, tensors, ops) -> None:
        for prefix, part in self.children():
            own = {k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}
            part.bind(own, ops)

    def forward(self, ctx, x, delta, cache: LayerCache):
        h = self.norm1.forward(ctx, x, delta)
        delta = self.mixer.forward(ctx, h, cache)
        h = self.norm2.forward(ctx, x, delta)
        delta = self.ffn.forward(ctx, h)
        return x, delta
