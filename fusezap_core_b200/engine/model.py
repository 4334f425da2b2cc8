"""The model: parts built from a `ModelSpec`, bound to loaded tensors. It holds no sizes of its own.

`load_model(path, dtype, device, max_len)` mirrors the reference's entry (fusezap/serve/models/__init__.py:9-13):
config.json -> registry -> parts -> safetensors by name. The output matrix is the stored one unless the model ties its
embeddings or the checkpoint has none, then the embedding table (fusezap/serve/models/llama.py:362-367).
"""
from __future__ import annotations
from dataclasses import replace
from typing import Any

import torch

from ..cache import KVNeed
from ..config import ModelSpec, describe, read_config_json
from ..parts import BLOCKS, FEED_FORWARDS, LOGIT_TRANSFORMS, MIXERS, NORMS, POSITIONS, build
from ..weights import ParamSpec, load_weights
from ..weights.loader import TORCH_DTYPE


def build_layers(spec: ModelSpec) -> list[Any]:
    layers = []
    for ls in spec.layers:
        mixer = build(MIXERS, "mixer", ls.mixer)
        ffn = build(FEED_FORWARDS, "feed-forward", ls.ffn)
        if ls.block.kind not in BLOCKS:
            raise NotImplementedError(f"block kind {ls.block.kind!r} is not registered (have {sorted(BLOCKS)})")
        layers.append(BLOCKS[ls.block.kind](mixer, ffn, _norm_maker(ls), **ls.block.params))
    return layers


def _norm_maker(ls):
    """What a block builds its norms with: the spec it names, else the layer's fallback kind."""
    def make_norm(spec=None):
        spec = spec if spec is not None else ls.norm
        if spec is None:
            raise ValueError(f"layer {ls.prefix!r}: the block asks for a norm that neither its params nor the layer's "
                             f"`norm` describe")
        return build(NORMS, "norm", spec)
    return make_norm


def declared_tensors(spec: ModelSpec, layers: list[Any] | None = None) -> dict[str, ParamSpec]:
    """Every tensor name the model reads, in a fixed order, with its shape. Optional groups get the layer's prefix."""
    layers = layers if layers is not None else build_layers(spec)
    out: dict[str, ParamSpec] = {spec.embed_name: ParamSpec((spec.vocab_size, spec.hidden_size))}
    for ls, block in zip(spec.layers, layers):
        for k, p in block.tensors().items():
            out[ls.prefix + k] = replace(p, group=ls.prefix + p.group) if p.group else p
    final = build(NORMS, "norm", spec.final_norm)
    stem = spec.final_norm_name.rsplit(".", 1)[0]
    for k, p in final.tensors().items():
        out[f"{stem}.{k}"] = p
    if spec.lm_head_name:
        out[spec.lm_head_name] = ParamSpec((spec.vocab_size, spec.hidden_size), group="lm_head", ignore=spec.tie_embeddings)
    return out


def optional_groups_to_write(typed: Any, spec: ModelSpec) -> set[str]:
    expected = declared_tensors(spec)
    if hasattr(typed, "random_optional_groups"):
        return set(typed.random_optional_groups(expected))
    return set() if spec.tie_embeddings else {"lm_head"}


class DecoderModel:
    def __init__(self, spec: ModelSpec, typed: Any = None):
        spec.validate()
        self.spec, self.config = spec, typed
        self.layers = build_layers(spec)
        self.final_norm = build(NORMS, "norm", spec.final_norm)
        self.positions = {name: build(POSITIONS, "position encoding", p) for name, p in spec.positions.items()}
        self.logit_transform = (build(LOGIT_TRANSFORMS, "logit transform", spec.logit_transform)
                                if spec.logit_transform is not None else None)
        self.embed_scale = 1.0 if spec.embed_scale is None else float(spec.embed_scale)
        for n, e in enumerate(spec.schedule):
            pn = self.layers[e.layer].mixer.position_name()
            if pn is not None and pn not in self.positions:
                raise ValueError(f"layer {e.layer} names position encoding {pn!r}, the model has {sorted(self.positions)}")
        self.embed: torch.Tensor | None = None
        self.lm_head: torch.Tensor | None = None
        self.dtype: str | None = None
        self.device: torch.device | None = None
        self.max_len = 0

    # ---- what the cache manager must provide
    def cache_needs(self) -> dict[int, KVNeed]:
        needs: dict[int, KVNeed] = {}
        for e in self.spec.schedule:
            need = self.layers[e.layer].mixer.cache_need()
            if need is None:
                continue
            if e.cache in needs and needs[e.cache] != need:
                raise ValueError(f"cache slot {e.cache} is used by layers with different needs: {needs[e.cache]} and {need}")
            needs[e.cache] = need
        return needs

    def state_needs(self) -> dict[tuple[int, str], Any]:
        """(schedule entry, name) -> what the mixer declares: a shape (float32), or (shape, torch dtype)."""
        return {(n, name): need for n, e in enumerate(self.spec.schedule)
                for name, need in self.layers[e.layer].mixer.state_need().items()}

    def graph_safe(self) -> bool:
        """True if every part's forward is a fixed sequence of kernels over device data (see `Part.graph_safe`)."""
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def parts(self) -> list[Any]:
        """Every part of the model, blocks and what they hold included, each once."""
        out, seen = [], set()
        stack = [self.final_norm, *self.positions.values(), *self.layers]
        if self.logit_transform is not None:
            stack.append(self.logit_transform)
        while stack:
            p = stack.pop()
            if id(p) in seen:
                continue
            seen.add(id(p))
            out.append(p)
            children = getattr(p, "children", None)
            if children is not None:
                stack += [c for _, c in children()]
            for name in ("mixer", "ffn"):          # a block that does not list its children still has these two
                if hasattr(p, name):
                    stack.append(getattr(p, name))
        return out

    def expected_tensors(self) -> dict[str, ParamSpec]:
        return declared_tensors(self.spec, self.layers)

    # ---- tensors in
    def bind(self, tensors: dict[str, torch.Tensor], ops: Any, dtype: str, device: torch.device, max_len: int) -> "DecoderModel":
        spec = self.spec
        self.dtype, self.device, self.max_len = dtype, torch.device(device), max_len
        self.embed = tensors[spec.embed_name]
        head = None if spec.tie_embeddings or not spec.lm_head_name else tensors.get(spec.lm_head_name)
        self.lm_head = head if head is not None else self.embed
        for ls, block in zip(spec.layers, self.layers):
            block.bind({k[len(ls.prefix):]: v for k, v in tensors.items() if k.startswith(ls.prefix)}, ops)
        stem = spec.final_norm_name.rsplit(".", 1)[0] + "."
        self.final_norm.bind({k[len(stem):]: v for k, v in tensors.items() if k.startswith(stem)}, ops)
        for p in self.positions.values():
            p.prepare(max_len, self.device)
        return self

    def generate(self, prompt_ids: list[int], max_tokens: int = 16, params: Any = None, stop_token_ids: list[int] | None = None,
                 block_size: int = 16) -> list[int]:
        """One prompt in, its new tokens out: the batch-1 convenience of the reference's model class
        (fusezap/serve/models/llama.py:916-929). Builds a one-request engine with just enough pages; `params` (a
        SamplingParams) overrides max_tokens / stop_token_ids; greedy by default."""
        from ..sampling import SamplingParams
        from .llm_engine import LLMEngine
        if params is None:
            params = SamplingParams(max_tokens=max_tokens, stop_token_ids=list(stop_token_ids or []))
        need = len(prompt_ids) + params.max_tokens
        if need > self.max_len:
            raise ValueError(f"prompt ({len(prompt_ids)}) + max_tokens ({params.max_tokens}) exceeds the length the model "
                             f"was loaded for ({self.max_len})")
        eng = LLMEngine(self, num_blocks=-(-need // block_size) + 1, block_size=block_size, max_num_seqs=1,
                        max_model_len=self.max_len)
        return eng.generate([prompt_ids], params)[0]

    def weight_bytes(self) -> int:
        """Bytes of every distinct tensor a step reads once (the decode roofline's weight term): each part says which
        tensors it reads (`Part.weight_tensors()`); the embedding table is not among them (a step gathers a few rows)
        unless it also serves as the output matrix."""
        seen: dict[int, int] = {}
        for part in self.parts():
            for t in part.weight_tensors():
                seen[t.data_ptr()] = t.numel() * t.element_size()
        if self.lm_head is not None:
            seen[self.lm_head.data_ptr()] = self.lm_head.numel() * self.lm_head.element_size()
        return sum(seen.values())


def load_model(path: str, dtype: str = "bfloat16", device: str | torch.device = "cuda:0", max_len: int | None = None,
               ops: Any = None) -> DecoderModel:
    """A model folder (config.json + safetensors) -> a bound model. `ops`: the kernel table; default: the CUDA kernels
    of `dtype` (building them at the first call), which refuse to run anywhere but on a GPU."""
    if dtype not in TORCH_DTYPE:
        raise ValueError(f"dtype {dtype!r} is not one of {sorted(TORCH_DTYPE)}")
    typed, spec = describe(read_config_json(path))
    model = DecoderModel(spec, typed)
    if ops is None:
        from ..kernels import cuda_ops
        ops = cuda_ops(dtype, device)
    tensors = load_weights(path, model.expected_tensors(), device, dtype)
    model.ops = ops
    return model.bind(tensors, ops, dtype, torch.device(device), max_len or spec.max_position)


def random_model(config: dict, dtype: str = "bfloat16", device: str | torch.device = "cuda:0", seed: int = 0,
                 max_len: int | None = None, ops: Any = None, norm_noise: bool = False) -> DecoderModel:
    """A bound model with seeded random weights drawn on the device (no files): matrices and biases N(0, 0.02), norm
    weights 1 (or 1 + N(0, 0.02)). The same rule as the random-weights writer, from the device's own generator, for
    models too large to write and read back quickly."""
    if dtype not in TORCH_DTYPE:
        raise ValueError(f"dtype {dtype!r} is not one of {sorted(TORCH_DTYPE)}")
    typed, spec = describe(config)
    model = DecoderModel(spec, typed)
    device = torch.device(device)
    if ops is None:
        from ..kernels import cuda_ops
        ops = cuda_ops(dtype, device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    compute = TORCH_DTYPE[dtype]
    groups = optional_groups_to_write(typed, spec)
    tensors: dict[str, torch.Tensor] = {}
    for name, p in model.expected_tensors().items():
        if p.ignore or (p.group is not None and p.group not in groups):
            continue
        if p.role == "int_table":
            tensors[name] = torch.zeros(p.shape, dtype=torch.int32, device=device)
            continue
        if p.init == "ones":
            t = torch.ones(p.shape, dtype=torch.float32, device=device)
            if norm_noise:
                t += torch.randn(p.shape, generator=gen, dtype=torch.float32, device=device) * 0.02
        elif p.init == "zeros":
            t = torch.zeros(p.shape, dtype=torch.float32, device=device)
        else:
            t = torch.empty(p.shape, dtype=compute, device=device)
            t.normal_(0.0, 0.02, generator=gen)
        tensors[name] = t.to(torch.float32 if (p.role == "vector" and compute != torch.float32) else compute)
    model.ops = ops
    return model.bind(tensors, ops, dtype, device, max_len or spec.max_position)
