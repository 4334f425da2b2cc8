"""Architecture-independent description of a decoder: what the engine builds and runs.

An architecture (one entry of the registry) turns its own config.json into a `ModelSpec`. Everything below the registry
(the weight loader, the cache manager, the step function, the scheduler) reads only this description, never a
model-specific config class, so another architecture is a new function that returns a `ModelSpec`.

  ModelSpec
    layers:   list[LayerSpec]      distinct layers (each owns weights); a layer names its parts by kind + parameters
    schedule: list[ScheduleEntry]  the order in which layers run; an entry may name a layer that an earlier entry already
                                   named (shared weights, own cache), or read another entry's cache instead of writing one
    positions: dict[str, PartSpec] position encodings by name (a mixer refers to one by name)
"""
from __future__ import annotations
from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by `kind` (a name in the parts registry) with its sizes and constants as `params`."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)

    def __hash__(self) -> int:  # params is a dict; identity of a spec is its printed form
        return hash((self.kind, repr(sorted(self.params.items()))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how its parts are arranged (`block`), and the parts. `prefix` is the layer's tensor-name prefix.
    Norms belong to the block: it decides how many it has, where they stand and what they are called, and its params
    may name a spec for each (any number, any kinds). `norm` is only the kind a block falls back on for a norm that its
    params leave open; a layer whose block names all its norms needs none."""
    prefix: str
    block: PartSpec
    mixer: PartSpec
    ffn: PartSpec
    norm: PartSpec | None = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer. `cache` is the cache slot the mixer uses: entries with the same `cache` share keys and
    values; `write_cache=False` means this execution only reads what the slot's owner wrote earlier in the same step."""
    layer: int
    cache: int
    write_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embed_name: str
    lm_head_name: str | None          # the output matrix; None: the model has none of its own
    tie_embeddings: bool              # True: logits use the embedding table, `lm_head_name` is ignored if present;
                                      # False: `lm_head_name` is used when the checkpoint has it, else the embedding
    final_norm: PartSpec
    final_norm_name: str
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    positions: dict[str, PartSpec]
    max_position: int
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    embed_scale: float | None = None          # embeddings are multiplied by this (in float32) as they are gathered
    logit_transform: PartSpec | None = None   # a part (kind in the logit-transform registry) applied to the float32
                                              # logits of the wanted rows, in place, before anything reads them

    def validate(self) -> None:
        if self.hidden_size <= 0 or self.vocab_size <= 0:
            raise ValueError(f"hidden_size and vocab_size must be positive, got {self.hidden_size}, {self.vocab_size}")
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        owners: dict[int, int] = {}
        for n, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {n} names layer {e.layer}, the model has {len(self.layers)}")
            if e.write_cache:
                if e.cache in owners:
                    raise ValueError(f"schedule entries {owners[e.cache]} and {n} both write cache slot {e.cache}")
                owners[e.cache] = n
            elif e.cache not in owners:
                raise ValueError(f"schedule entry {n} reads cache slot {e.cache} before any entry wrote it")
        if not self.schedule:
            raise ValueError("the schedule is empty")
