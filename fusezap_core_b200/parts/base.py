"""The interfaces of the parts a layer is put together from, and the registries that map a part's `kind` to its class.

A part is built from `PartSpec.params` only (its sizes and constants); it never learns which model it is in. It says
which tensors it needs (`tensors()`: names relative to the part, with shapes), receives them (`bind`), and computes
through the kernel table of the step (`ctx.ops`), taking scratch buffers from `ctx.ws`.

  Mixer.forward(ctx, h, cache)  -> delta     h: (N, D) activation dtype; delta: (N, D) float32, added to the residual
  FeedForward.forward(ctx, h)   -> delta
  Norm.forward(ctx, x, delta, rows=None) -> h   x: (N, D) float32 residual stream, updated in place with `+ delta`
                                                (rows given: only those rows are normed and x is left as it is)
  PositionEncoding.prepare(max_len, device)      builds its tables
  PositionEncoding.rotate_and_store(ctx, qkv, q_out, cache, num_heads, num_kv_heads, head_dim)
  Block.forward(ctx, x, delta, cache) -> (x, delta)   the arrangement of norms, mixer and feed-forward of one layer
  LogitTransform.forward(ctx, logits) -> None    changes the float32 logits of the wanted rows in place

Register a new part with `@register_mixer("name")` (or _feed_forward, _norm, _position, _block, _logit_transform) and name it in a
`PartSpec`; nothing else in the package changes.
"""
from __future__ import annotations
from dataclasses import dataclass, field
from typing import Any, Callable, TYPE_CHECKING

import torch

from ..cache import KVNeed
from ..config import PartSpec
from ..weights import ParamSpec

if TYPE_CHECKING:  # pragma: no cover
    from ..engine.step import StepContext

MIXERS: dict[str, type] = {}
FEED_FORWARDS: dict[str, type] = {}
NORMS: dict[str, type] = {}
POSITIONS: dict[str, type] = {}
BLOCKS: dict[str, type] = {}
LOGIT_TRANSFORMS: dict[str, type] = {}


def _register(table: dict[str, type], what: str) -> Callable[[str], Callable[[type], type]]:
    def named(name: str) -> Callable[[type], type]:
        def put(cls: type) -> type:
            table[name] = cls
            return cls
        return put
    named.__doc__ = f"Class decorator: register a {what} under a kind name."
    return named


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position = _register(POSITIONS, "position encoding")
register_block = _register(BLOCKS, "block")
register_logit_transform = _register(LOGIT_TRANSFORMS, "logit transform")


def build(table: dict[str, type], what: str, spec: PartSpec) -> Any:
    if spec.kind not in table:
        raise NotImplementedError(f"{what} kind {spec.kind!r} is not registered (have {sorted(table)})")
    return table[spec.kind](**spec.params)


@dataclass
class LayerCache:
    """What one schedule entry's mixer sees of the cache manager."""
    keys: torch.Tensor | None = None        # (pages, Hkv, page_size, hd) view of this entry's cache slot
    values: torch.Tensor | None = None
    group: int = -1                         # index of the block-table set in the step metadata
    page_size: int = 0
    write: bool = True                      # False: read what the slot's owner wrote earlier in this step
    state: dict[str, torch.Tensor] = field(default_factory=dict)   # name -> (num_slots, *shape) float32


class Part:
    # False for a part whose forward depends on the step's host-side metadata (for instance a Python loop over
    # `ctx.meta.segments`): such a step cannot be replayed from a captured CUDA graph, and the engine then runs every
    # step kernel by kernel.
    graph_safe = True

    def tensors(self) -> dict[str, ParamSpec]:
        return {}

    def bind(self, tensors: dict[str, torch.Tensor], ops: Any) -> None:
        """Receives the tensors of `tensors()` that the checkpoint has (optional ones may be absent)."""

    def weight_tensors(self) -> list[torch.Tensor]:
        """Every device tensor a step reads once for this part (sub-parts not included): what the decode roofline counts
        as this part's weight bytes. The default finds the tensors the part keeps as attributes (alone, or in tuples
        and lists); a part that keeps them elsewhere (a dict, a nested object) overrides this."""
        found = []
        for v in vars(self).values():
            if isinstance(v, torch.Tensor):
                found.append(v)
            elif isinstance(v, (tuple, list)):
                found += [t for t in v if isinstance(t, torch.Tensor)]
        return found


class Mixer(Part):
    def cache_need(self) -> KVNeed | None:
        return None

    def state_need(self) -> dict[str, Any]:
        """Per-request state of fixed size: {name: shape} (float32) or {name: (shape, torch dtype)}."""
        return {}

    def position_name(self) -> str | None:
        return None

    def step_needs(self) -> tuple[str, ...]:
        """Kinds of per-step data this mixer's kernels need beside the common metadata (for instance "attention": the
        kernel table then plans its attention kernels' tiles for every step). None by default."""
        return ()

    def forward(self, ctx: "StepContext", h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx: "StepContext", h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(self, ctx: "StepContext", x: torch.Tensor, delta: torch.Tensor | None,
                rows: torch.Tensor | None = None, n_rows: int | None = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, max_len: int, device: torch.device) -> None:
        raise NotImplementedError

    def rotate_and_store(self, ctx: "StepContext", qkv: torch.Tensor, q_out: torch.Tensor, cache: LayerCache,
                         num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        raise NotImplementedError

    def project_rotate_store(self, ctx: "StepContext", h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None,
                             q_out: torch.Tensor, cache: LayerCache, num_heads: int, num_kv_heads: int,
                             head_dim: int) -> bool:
        """Optional: the mixer's q/k/v product (h . w^T + bias) and `rotate_and_store` as one operation. False (the
        default) means nothing was done and the mixer runs the product and `rotate_and_store` itself."""
        return False


class Block(Part):
    """Arranges norm(s), mixer and feed-forward. Built with the already built parts of its layer and `make_norm(spec)`,
    which builds a norm from a `PartSpec` (None: the layer's fallback norm kind); `children()` lists (tensor-name
    prefix, part) of everything it holds."""
    def children(self) -> tuple:
        return ()

    def forward(self, ctx: "StepContext", x: torch.Tensor, delta: torch.Tensor | None,
                cache: LayerCache) -> tuple[torch.Tensor, torch.Tensor | None]:
        raise NotImplementedError


class LogitTransform(Part):
    """Changes the logits of the wanted rows, (R, vocab) float32, in place (a soft cap, a scale, a bias...). With one in
    the model the output product always writes its logits (no fused argmax)."""
    def forward(self, ctx: "StepContext", logits: torch.Tensor) -> None:
        raise NotImplementedError
