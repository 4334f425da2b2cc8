"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a configuration and a seed.

Every matrix and bias is drawn N(0, 0.02), norm weights are 1 (or 1 + N(0, 0.02) with `norm_noise`), tensor names are
the checkpoint's own; a tied model writes no output matrix. The reference's generator tiles one random block into every
shape and always writes an untied head (fusezap/serve/models/random_weights.py:28-54); this one draws each tensor from
one `numpy.random.default_rng(seed)` stream in the order the model declares its tensors, so a seed names one model
whatever dtype it is stored in (bfloat16 is the round-to-nearest-even of the float32 draw).
"""
from __future__ import annotations
import json
import os
from typing import Iterator

import numpy as np
import torch

from ..config import describe
from .params import ParamSpec
from .safetensors_io import write_file

STD = 0.02


def draw(rng: np.random.Generator, p: ParamSpec, norm_noise: bool, optional: bool) -> torch.Tensor:
    if p.role == "int_table":
        return torch.zeros(p.shape, dtype=torch.int32)
    if p.init == "ones":
        a = np.ones(p.shape, np.float32)
        if norm_noise:
            a = a + rng.standard_normal(p.shape, dtype=np.float32) * np.float32(STD)
    elif p.init == "zeros":
        a = np.zeros(p.shape, np.float32)
    else:
        a = rng.standard_normal(p.shape, dtype=np.float32) * np.float32(STD)
    return torch.from_numpy(a)


def random_tensors(expected: dict[str, ParamSpec], seed: int, dtype: str = "float32", norm_noise: bool = False,
                   optional_groups: set[str] | None = None, std_scale: float = 1.0) -> Iterator[tuple[str, torch.Tensor]]:
    """Yields (name, tensor) in declaration order. Optional groups are written only if named in `optional_groups`."""
    rng = np.random.default_rng(seed)
    td = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    for name, p in expected.items():
        if p.ignore or (p.group is not None and p.group not in (optional_groups or ())):
            continue
        t = draw(rng, p, norm_noise, p.group is not None)
        if std_scale != 1.0 and p.init == "normal" and p.role != "int_table":
            t = t * std_scale
        yield name, (t if p.role == "int_table" else t.to(td))


def write_random_model(config: dict, out_dir: str, seed: int, dtype: str = "float32", norm_noise: bool = False,
                       std_scale: float = 1.0) -> str:
    """config: a config.json dict of a registered architecture. Returns out_dir."""
    from ..engine.model import declared_tensors, optional_groups_to_write
    typed, spec = describe(config)
    expected = declared_tensors(spec)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    write_file(os.path.join(out_dir, "model.safetensors"),
               random_tensors(expected, seed, dtype, norm_noise, optional_groups_to_write(typed, spec), std_scale))
    return out_dir
