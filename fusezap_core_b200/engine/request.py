"""A request as the engine keeps it: its tokens, how many of them are in the cache, and where it stands.

The engine never distinguishes "prompt phase" from "decode phase" by a flag. A request *knows* tokens (its prompt, then
what was generated) and has some of them *cached* (their keys and values are in its pages). What is known but not cached
is *pending* and is what the next steps run: the whole prompt of a new request, one token of a request that generates,
everything known of a request that lost its pages. This one notion covers prefill, chunked prefill, decode and
recomputation after an eviction.
"""
from __future__ import annotations
import enum
from dataclasses import dataclass, field
from typing import Any


class Phase(enum.Enum):
    QUEUED = "queued"      # waits for admission (new, or evicted and to be recomputed); holds no pages
    LIVE = "live"          # admitted: holds pages and takes part in steps
    DONE = "done"          # ended; holds nothing


@dataclass(eq=False)
class Request:
    rid: int
    prompt: list[int]
    params: Any                     # SamplingParams (the scheduler reads nothing of it)
    order: int                      # arrival number: the smaller, the more senior
    sampler: Any = None
    generated: list[int] = field(default_factory=list)
    cached: int = 0                 # known tokens whose keys and values are in the cache
    phase: Phase = Phase.QUEUED
    ended_by: str | None = None     # "stop" | "length" | "abort"
    evictions: int = 0
    evicted_in: int = -1            # scheduler step of the last eviction
    admitted_in: int = -1           # scheduler step that first admitted it
    ended_in: int = -1

    @property
    def known(self) -> int:
        return len(self.prompt) + len(self.generated)

    @property
    def pending(self) -> int:
        return self.known - self.cached

    @property
    def decoding(self) -> bool:
        """One token to run, and not the first one: a row of a decode step."""
        return self.cached > 0 and self.known - self.cached == 1

    @property
    def history(self) -> list[int]:
        return self.prompt + self.generated

    def token(self, i: int) -> int:
        n = len(self.prompt)
        return self.prompt[i] if i < n else self.generated[i - n]

    def span(self, lo: int, hi: int) -> list[int]:
        """Known tokens lo .. hi-1."""
        n = len(self.prompt)
        if hi <= n:
            return self.prompt[lo:hi]
        if lo >= n:
            return self.generated[lo - n: hi - n]
        return self.prompt[lo:] + self.generated[: hi - n]
