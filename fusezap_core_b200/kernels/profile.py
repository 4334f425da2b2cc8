"""A per-step profile by kernel class: launches, device time, and the bytes each class had to move at least.

The reference has a switch that times the phases of a serving step (fusezap/serve/stepprof.py:1-86); here the unit is
the kernel class (embed, norm, linear, rotation + cache write, attention, ...). With `EngineConfig(profile=True)` (or
`--profile`) every step runs kernel by kernel (no CUDA graphs, no launching ahead) and the kernel table records a CUDA
event after every launch; the time between two consecutive events of a step is booked to the later one's class. That
includes the gap before the kernel starts, so classes of many short kernels read a little high; the shares are what
the table is for. `ideal_bytes` is what the class must read and write at least (weights once, activations once, the
keys and values a row may see), so `bytes / time` against the copy bandwidth says how far a class is from its roofline.
"""
from __future__ import annotations
from collections import OrderedDict
from typing import Any, Iterable


class StepProfile:
    """Collects (class, event, ideal bytes) per launch; `marks` are event-like objects with `elapsed_time(other)`."""
    def __init__(self, make_event):
        self._make_event = make_event
        self._chain: list[tuple[str, Any, int]] = []       # of the current step; the first entry is the step's start
        self._done: list[list[tuple[str, Any, int]]] = []
        self.totals: "OrderedDict[str, dict]" = OrderedDict()
        self.steps = 0

    def begin_step(self) -> None:
        self._flush()
        ev = self._make_event()
        ev.record()
        self._chain = [("(start)", ev, 0)]

    def note(self, what: str, ideal_bytes: int = 0) -> None:
        if not self._chain:
            self.begin_step()
        ev = self._make_event()
        ev.record()
        self._chain.append((what, ev, int(ideal_bytes)))

    def _flush(self) -> None:
        if len(self._chain) > 1:
            self._done.append(self._chain)
        self._chain = []

    def collect(self, synchronize) -> None:
        """Turns the recorded events into totals (waits for the device first)."""
        self._flush()
        if not self._done:
            return
        synchronize()
        for chain in self._done:
            self.steps += 1
            for (_, before, _), (what, after, nbytes) in zip(chain, chain[1:]):
                t = self.totals.setdefault(what, {"launches": 0, "ms": 0.0, "ideal_bytes": 0})
                t["launches"] += 1
                t["ms"] += float(before.elapsed_time(after))
                t["ideal_bytes"] += nbytes
        self._done = []

    def report(self) -> dict:
        total = sum(t["ms"] for t in self.totals.values()) or 1.0
        rows = []
        for what, t in self.totals.items():
            gbs = t["ideal_bytes"] / (t["ms"] * 1e-3) / 1e9 if t["ms"] > 0 and t["ideal_bytes"] else None
            rows.append({"class": what, "launches": t["launches"], "ms": round(t["ms"], 4),
                         "share": round(t["ms"] / total, 4), "ideal_bytes": t["ideal_bytes"],
                         "ideal_gbs": None if gbs is None else round(gbs, 1)})
        rows.sort(key=lambda r: -r["ms"])
        return {"steps": self.steps, "ms": round(total, 4), "classes": rows}


def format_report(rep: dict) -> str:
    lines = [f"profile: {rep['steps']} steps, {rep['ms']:.3f} ms on the device",
             f"  {'class':<34}{'launches':>9}{'ms':>11}{'share':>8}{'ideal MB':>11}{'GB/s':>9}"]
    for r in rep["classes"]:
        gbs = "" if r["ideal_gbs"] is None else f"{r['ideal_gbs']:.0f}"
        lines.append(f"  {r['class']:<34}{r['launches']:>9}{r['ms']:>11.3f}{100 * r['share']:>7.1f}%"
                     f"{r['ideal_bytes'] / 1e6:>11.1f}{gbs:>9}")
    return "\n".join(lines)


def ideal_linear_bytes(m: int, n: int, k: int, in_size: int, w_size: int, out_size: int) -> int:
    return m * k * in_size + n * k * w_size + m * n * out_size


def contexts(segments: Iterable[Any]) -> int:
    """Keys the rows of a step may see in all: a row at position p sees p + 1 keys."""
    total = 0
    for s in segments:
        total += s.n * s.pos0 + s.n * (s.n + 1) // 2
    return total
