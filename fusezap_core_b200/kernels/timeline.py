"""Reads the per-launch timestamps that libraries built with `-DFZ_TIMELINE` keep (a measurement aid: set
`FZB200_NVCC_EXTRA=-DFZ_TIMELINE` before the libraries are first built or loaded).

Every launch leaves two numbers of the GPU's global timer: when thread 0 of its first block started, and when that
thread's wait on the kernels before it returned. The difference between two successive launches' second numbers is what
the earlier kernel costs on the critical path of the step; second minus first says how long before its dependency was
met a kernel's first block was already resident (programmatic dependent launch at work).
"""
from __future__ import annotations
import ctypes

import numpy as np

_FILES = (("core", ("rowwise", "gemm_simt", "attn_simt")), ("tc", ("gemm_tc", "attn_decode", "attn_prefill", "attn_prefill_tc")))
SLOTS = 4096


def read(ops) -> list[tuple[int, int, str]]:
    """(start ns, dependency met ns, source file) of every launch since the last call, in order of start; clears the
    buffers. Raises if the libraries were built without the switch."""
    out = []
    for attr, names in _FILES:
        lib = getattr(ops, attr, None)
        if lib is None:
            continue
        for name in names:
            try:
                fn = getattr(lib, "fz_timeline_" + name)
            except AttributeError:
                raise RuntimeError("the kernel libraries were built without -DFZ_TIMELINE (set FZB200_NVCC_EXTRA before "
                                   "they are built)") from None
            buf = (ctypes.c_ulonglong * (2 * SLOTS))()
            n = ctypes.c_uint(0)
            status = fn(buf, ctypes.byref(n))
            if status != 0:
                raise RuntimeError(f"fz_timeline_{name}: CUDA error {status}")
            a = np.frombuffer(buf, dtype=np.uint64).reshape(-1, 2)[: min(n.value, SLOTS)]
            out += [(int(s), int(d), name) for s, d in a]
    return sorted(out)


def per_launch_costs(events: list[tuple[int, int, str]], launches_per_step: int) -> list[dict]:
    """Medians over the steps in `events` (a whole number of steps of `launches_per_step` launches each), per position in
    the step: the source file, the critical-path cost in us (to the next launch's met dependency) and how long the first
    block was resident before its own dependency was met."""
    steps = len(events) // launches_per_step
    rows = []
    for i in range(launches_per_step):
        cost, early = [], []
        for s in range(steps):
            e = events[s * launches_per_step + i]
            nxt = s * launches_per_step + i + 1
            if nxt < len(events) and (i + 1 < launches_per_step):
                cost.append((events[nxt][1] - e[1]) / 1e3)
            early.append((e[1] - e[0]) / 1e3)
        rows.append({"file": events[i][2], "cost_us": float(np.median(cost)) if cost else float("nan"),
                     "resident_before_us": float(np.median(early))})
    return rows
