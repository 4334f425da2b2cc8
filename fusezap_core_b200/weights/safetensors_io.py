"""The safetensors container, read and written without any package: 8-byte little-endian header length, a JSON header
`{name: {dtype, shape, data_offsets}}` (`__metadata__` ignored), then the raw little-endian bytes
(format as the reference reads it: fusezap/serve/weights.py:16-39). A model folder is one file, or the shards that
`model.safetensors.index.json` lists, or every `*.safetensors` in it (weights.py:132-147).

Tensors come back as torch CPU tensors that view one read-only memory map per file (nothing is copied until a tensor is
moved or converted). BF16 is viewed as `torch.bfloat16`.
"""
from __future__ import annotations
import json
import os
import struct
from typing import Iterable

import numpy as np
import torch

_NP = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64, "I32": np.int32,
       "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_}
_TORCH_TO_ST = {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
                torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8",
                torch.bool: "BOOL"}


class SafetensorsError(ValueError):
    pass


def read_header(path: str) -> tuple[dict, int]:
    """(header without __metadata__, byte offset of the data section)."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) < 8:
            raise SafetensorsError(f"{path}: shorter than a safetensors header")
        (n,) = struct.unpack("<Q", raw)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit a file of {size} bytes")
        try:
            header = json.loads(f.read(n))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: the header is not JSON ({e})") from None
    header.pop("__metadata__", None)
    for name, v in header.items():
        if v.get("dtype") not in _NP:
            raise SafetensorsError(f"{path}: tensor {name!r} has unknown dtype {v.get('dtype')!r}")
        s, e = v["data_offsets"]
        want = int(np.prod(v["shape"], dtype=np.int64)) * np.dtype(_NP[v["dtype"]]).itemsize
        if e - s != want or s < 0 or 8 + n + e > size:
            raise SafetensorsError(f"{path}: tensor {name!r} spans bytes [{s}, {e}) but its shape {v['shape']} "
                                   f"needs {want}, in a data section of {size - 8 - n}")
    return header, 8 + n


def read_file(path: str) -> dict[str, torch.Tensor]:
    header, base = read_header(path)
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    out: dict[str, torch.Tensor] = {}
    for name, v in header.items():
        s, e = v["data_offsets"]
        a = mm[base + s: base + e].view(_NP[v["dtype"]]).reshape(v["shape"])
        with _quiet_readonly():
            t = torch.from_numpy(a)
        out[name] = t.view(torch.bfloat16) if v["dtype"] == "BF16" else t
    return out


class _quiet_readonly:
    """torch warns that a read-only array is not writable; these tensors are only ever read."""
    def __enter__(self):
        import warnings
        self._c = warnings.catch_warnings()
        self._c.__enter__()
        warnings.simplefilter("ignore", UserWarning)
    def __exit__(self, *a):
        return self._c.__exit__(*a)


def model_files(model_dir: str) -> list[str]:
    if os.path.isfile(model_dir):
        return [model_dir]
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            wm = json.load(f)["weight_map"]
        return [os.path.join(model_dir, s) for s in sorted(set(wm.values()))]
    fns = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if not fns:
        raise FileNotFoundError(f"no .safetensors files in {model_dir!r}")
    return [os.path.join(model_dir, f) for f in fns]


def read_model_dir(model_dir: str) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}
    for fn in model_files(model_dir):
        if not os.path.isfile(fn):
            raise FileNotFoundError(f"{fn!r} is listed by the index but does not exist")
        out.update(read_file(fn))
    return out


def write_file(path: str, tensors: Iterable[tuple[str, torch.Tensor]] | dict[str, torch.Tensor]) -> None:
    """Write tensors in the order given (a dict or an iterable of pairs; the iterable form lets a writer produce one
    tensor at a time). Data offsets are 8-byte aligned by padding the header with spaces."""
    items = list(tensors.items()) if isinstance(tensors, dict) else list(tensors)
    header: dict[str, dict] = {}
    off = 0
    for name, t in items:
        if t.dtype not in _TORCH_TO_ST:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_ST[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    raw = json.dumps(header, separators=(",", ":")).encode()
    raw += b" " * (-(8 + len(raw)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for _, t in items:
            t = t.detach().contiguous().cpu()
            a = t.view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.numpy()
            f.write(a.tobytes())
    os.replace(tmp, path)
