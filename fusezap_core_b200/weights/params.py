"""What a part says about each tensor it needs: shape, role and how the random-weights writer fills it."""
from __future__ import annotations
from dataclasses import dataclass


@dataclass(frozen=True)
class ParamSpec:
    shape: tuple[int, ...]
    role: str = "matrix"          # "matrix": cast to the compute dtype; "vector": a tensor stored in 32-bit stays so;
                                  # "int_table": kept as int32
    init: str = "normal"          # "normal" (std 0.02), "ones", "zeros"
    group: str | None = None      # None: required. Otherwise the name of an all-or-none group of optional tensors
    ignore: bool = False          # accepted if present, never loaded (a tied model's stored output matrix)
