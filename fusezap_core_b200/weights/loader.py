"""Loads a model folder's tensors by name, after checking all of them against what the model's parts declare.

One `WeightsError` lists everything that is wrong at once: missing tensors (also an optional group of which only some
are present), unexpected tensors, and wrong shapes. dtype policy: in float32 everything floating becomes float32; in
bfloat16 matrices become bfloat16 (round to nearest even), a 1-D tensor stored in 32-bit stays float32, integer tables
become int32. (The reference converts every tensor to the model dtype: fusezap/serve/models/llama.py:290,
fusezap/serve/weights.py:158-164; it reports a missing tensor as a bare KeyError.)
"""
from __future__ import annotations
import torch

from .params import ParamSpec
from .safetensors_io import read_model_dir

_FLOATS = (torch.float64, torch.float32, torch.float16, torch.bfloat16)
# Buffers that some exporters write beside the parameters and that no model reads (they are recomputed from config.json):
# a tensor whose name ends in one of these is passed over instead of being reported as unexpected. (The reference loads
# by name and ignores every extra tensor; here any other extra tensor is an error.)
NON_PARAMETER_SUFFIXES = ("rotary_emb.inv_freq",)
TORCH_DTYPE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


class WeightsError(ValueError):
    def __init__(self, missing: list[str], unexpected: list[str], wrong: list[str], where: str = ""):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        def part(title: str, items: list[str]) -> str:
            return f"  {title} ({len(items)}): " + ", ".join(items) if items else ""
        lines = [p for p in (part("missing", missing), part("unexpected", unexpected), part("wrong shape or dtype", wrong)) if p]
        super().__init__(f"the tensors{' in ' + where if where else ''} do not match the model:\n" + "\n".join(lines))


def check_tensors(expected: dict[str, ParamSpec], found: dict[str, torch.Tensor], where: str = "") -> None:
    missing, wrong = [], []
    groups: dict[str, list[str]] = {}
    for name, p in expected.items():
        if p.group is not None:
            groups.setdefault(p.group, []).append(name)
        elif name not in found and not p.ignore:
            missing.append(name)
    for g, names in groups.items():
        have = [n for n in names if n in found]
        if have and len(have) != len(names):
            missing += [f"{n} (the others of optional group {g!r} are present)" for n in names if n not in found]
    for name, t in found.items():
        p = expected.get(name)
        if p is None or p.ignore:
            continue
        if tuple(t.shape) != tuple(p.shape):
            wrong.append(f"{name}: shape {tuple(t.shape)}, expected {tuple(p.shape)}")
        elif p.role == "int_table" and t.dtype in _FLOATS:
            wrong.append(f"{name}: dtype {t.dtype}, expected an integer table")
        elif p.role != "int_table" and t.dtype not in _FLOATS:
            wrong.append(f"{name}: dtype {t.dtype}, expected a floating-point tensor")
    unexpected = sorted(n for n in found if n not in expected and not n.endswith(NON_PARAMETER_SUFFIXES))
    if missing or unexpected or wrong:
        raise WeightsError(missing, unexpected, wrong, where)


def convert(t: torch.Tensor, role: str, compute_dtype: torch.dtype) -> torch.dtype:
    """The dtype a stored tensor is kept in."""
    if role == "int_table":
        return torch.int32
    if compute_dtype == torch.float32:
        return torch.float32
    if role == "vector" and t.dtype in (torch.float32, torch.float64):
        return torch.float32
    return compute_dtype


def load_weights(model_dir: str, expected: dict[str, ParamSpec], device: torch.device | str,
                 dtype: str) -> dict[str, torch.Tensor]:
    """{name: tensor on `device`} for every expected tensor that the folder has (optional ones may be absent)."""
    found = read_model_dir(model_dir)
    check_tensors(expected, found, where=repr(model_dir))
    compute = TORCH_DTYPE[dtype]
    out: dict[str, torch.Tensor] = {}
    for name, p in expected.items():
        if p.ignore or name not in found:
            continue
        t = found[name]
        out[name] = t.to(device=device, dtype=convert(t, p.role, compute)).contiguous()
    return out
