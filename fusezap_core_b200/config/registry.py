"""The one registry from an architecture's name (`model_type` in config.json) to its model description.

An architecture is a function `config.json dict -> (typed config, ModelSpec)`. `llama` and `qwen2` share one
(the reference maps both to one class too: fusezap/serve/models/__init__.py:6-8). An unknown name raises
NotImplementedError naming what is registered (models/__init__.py:12).
"""
from __future__ import annotations
import json
import os
from typing import Any, Callable

from .dense import DenseDecoderConfig
from .spec import ModelSpec

ArchitectureFn = Callable[[dict], tuple[Any, ModelSpec]]
ARCHITECTURES: dict[str, ArchitectureFn] = {}


def register_architecture(name: str, fn: ArchitectureFn | None = None):
    """Register `fn` under `name`; usable as a decorator. Registering a name twice replaces the entry."""
    def put(f: ArchitectureFn) -> ArchitectureFn:
        ARCHITECTURES[name] = f
        return f
    return put if fn is None else put(fn)


def _dense(c: dict) -> tuple[DenseDecoderConfig, ModelSpec]:
    cfg = DenseDecoderConfig.from_hf(c)
    return cfg, cfg.spec()


register_architecture("llama", _dense)
register_architecture("qwen2", _dense)


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{model_dir!r} has no config.json")
    with open(path) as f:
        config = json.load(f)
    # chat models stop on more ids than config.json lists: the ids of generation_config.json are merged in, as the
    # reference does (fusezap/serve/models/llama.py:443-451)
    gen = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gen):
        with open(gen) as f:
            more = json.load(f).get("eos_token_id")
        have = config.get("eos_token_id")
        ids = {*([have] if isinstance(have, int) else (have or [])), *([more] if isinstance(more, int) else (more or []))}
        if ids:
            config["eos_token_id"] = sorted(int(i) for i in ids)
    return config


def describe(config: dict) -> tuple[Any, ModelSpec]:
    """config.json dict -> (typed config, validated ModelSpec) through the registry."""
    name = config.get("model_type", "llama")
    if name not in ARCHITECTURES:
        raise NotImplementedError(f"model_type {name!r} is not supported (have {sorted(ARCHITECTURES)})")
    typed, spec = ARCHITECTURES[name](config)
    spec.validate()
    return typed, spec
