"""The cache manager: keys and values in pages with one block table per request and group, and fixed-size state slots.

Cache slots (one per schedule entry that writes a cache) with the same need (kv heads, head size, window) form a
*group*. A group has its own pages: one pool tensor `(slots, pages, 2, kv_heads, page_size, head_dim)` (keys at index
0, values at 1 of the third axis) and one block table per request, shared by the group's slots, so a page id means the
same page in every slot of the group (the reference keeps one table for all layers: fusezap/serve/kv_cache.py:436-460).
A full group keeps every page until the request ends; a window group gives back the pages that lie wholly before the
window of the request's next position (their table entries become -1) as soon as `commit` says how far the request is
computed. Position p of a request lives in page `table[p // page_size]` at offset `p % page_size`
(kv_cache.py:452-455).

Beside the pages there are `StateSlots`: per-request state of fixed size for mixers that declare some (the dense decoder
declares none). A request gets a slot with its first pages and returns it with them; a slot is zeroed when handed out.

All bookkeeping is on the host; device tensors are only allocated here, never computed on.
"""
from __future__ import annotations
from dataclasses import dataclass, field
from typing import Any, Hashable

import numpy as np
import torch

from .allocator import OutOfPages, PageAllocator


@dataclass(frozen=True)
class KVNeed:
    """What a mixer needs of the paged cache. window 0: all earlier keys; W: the last W keys (positions p-W+1 .. p)."""
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass
class KVGroup:
    need: KVNeed
    page_size: int
    num_pages: int
    slots: list[int]                              # cache slot ids that live in this group
    max_pages_per_request: int = 0
    pool: torch.Tensor | None = None              # (len(slots), num_pages, 2, Hkv, page_size, hd)
    allocator: PageAllocator = field(init=False)
    # request -> int32 row of page ids by page index (-1: given back, or not yet there) and how many entries are in use.
    # Entries below the first live page are -1; every entry from there to `lens[req]` holds a page.
    rows: dict[Hashable, np.ndarray] = field(default_factory=dict)
    lens: dict[Hashable, int] = field(default_factory=dict)

    def __post_init__(self) -> None:
        self.allocator = PageAllocator(self.num_pages)

    @property
    def tables(self) -> dict[Hashable, list[int]]:
        """The block tables as plain lists (for inspection and tests)."""
        return {r: self.rows[r][: self.lens[r]].tolist() for r in self.rows}

    def first_live_page(self, computed: int) -> int:
        """Index of the first page a query at position `computed` can still see."""
        if not self.need.window:
            return 0
        return max(0, computed - self.need.window + 1) // self.page_size

    def pages_needed(self, req: Hashable, computed: int, n_tokens: int) -> int:
        have = self.lens.get(req, 0)
        lo, hi = self.first_live_page(computed), -(-n_tokens // self.page_size)
        return max(0, hi - max(lo, have))      # everything between the first live page and `have` is already there

    def ensure(self, req: Hashable, computed: int, n_tokens: int) -> None:
        lo, hi = self.first_live_page(computed), -(-n_tokens // self.page_size)
        have = self.lens.get(req, 0)
        first = max(lo, have)
        if hi <= first and req in self.rows:
            return
        row = self.rows.get(req)
        if row is None or hi > row.shape[0]:
            grown = np.full(max(hi, self.max_pages_per_request, 1), -1, dtype=np.int32)
            if row is not None:
                grown[: row.shape[0]] = row
            row = self.rows[req] = grown
        if hi > first:
            row[first:hi] = self.allocator.allocate(hi - first)
        self.lens[req] = max(have, hi)

    def release_before(self, req: Hashable, computed: int) -> None:
        if not self.need.window or req not in self.rows:
            return
        row, lo = self.rows[req], min(self.first_live_page(computed), self.lens[req])
        head = row[:lo]
        gone = head[head >= 0]
        if gone.size:
            self.allocator.free(gone.tolist())
            head[:] = -1

    def free(self, req: Hashable) -> None:
        row = self.rows.pop(req, None)
        n = self.lens.pop(req, 0)
        if row is not None:
            held = row[:n]
            self.allocator.free(held[held >= 0].tolist())

    def view(self, slot: int) -> tuple[torch.Tensor, torch.Tensor]:
        """(keys, values) of one cache slot, each (num_pages, Hkv, page_size, hd) strided views of the pool."""
        s = self.pool[self.slots.index(slot)]
        return s[:, 0], s[:, 1]


def state_shape_dtype(need: Any) -> tuple[tuple[int, ...], torch.dtype]:
    """A mixer declares a piece of state as a shape (float32) or as (shape, torch dtype)."""
    if len(need) == 2 and isinstance(need[1], torch.dtype):
        return tuple(int(x) for x in need[0]), need[1]
    return tuple(int(x) for x in need), torch.float32


class StateSlots:
    """Slots of fixed size for per-request state. `tensors[(entry, name)]` is (num_slots, *shape) in the dtype the mixer
    declared (float32 unless it says otherwise)."""
    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self.owner: dict[Hashable, int] = {}
        self.tensors: dict[tuple[int, str], torch.Tensor] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self, req: Hashable) -> int:
        if req in self.owner:
            return self.owner[req]
        if not self._free:
            raise OutOfPages(f"no state slot free ({self.num_slots} in all)")
        s = self._free.pop()
        self.owner[req] = s
        for t in self.tensors.values():
            t[s].zero_()
        return s

    def release(self, req: Hashable) -> None:
        s = self.owner.pop(req, None)
        if s is not None:
            assert s not in self._free, f"state slot {s} freed twice"
            self._free.append(s)


class CacheManager:
    def __init__(self, needs: dict[int, KVNeed], state_needs: dict[tuple[int, str], tuple[int, ...]], page_size: int,
                 num_pages: int, max_requests: int, max_model_len: int, dtype: torch.dtype,
                 device: torch.device | str, allocate: bool = True):
        """needs: cache slot id -> KVNeed. state_needs: (schedule entry, name) -> shape of one request's state (float32),
        or (shape, torch dtype).
        num_pages is the page count of every group (a window group never needs more than a full one)."""
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.page_size, self.num_pages, self.max_model_len = page_size, num_pages, max_model_len
        self.max_pages_per_request = -(-max_model_len // page_size)
        self.dtype, self.device = dtype, torch.device(device)
        by_need: dict[KVNeed, list[int]] = {}
        for slot, need in sorted(needs.items()):
            by_need.setdefault(need, []).append(slot)
        self.groups: list[KVGroup] = [KVGroup(need, page_size, num_pages, slots, self.max_pages_per_request)
                                      for need, slots in by_need.items()]
        self.slot_group: dict[int, int] = {s: g for g, grp in enumerate(self.groups) for s in grp.slots}
        self.computed: dict[Hashable, int] = {}
        self.states = StateSlots(max_requests)
        if allocate:
            for grp in self.groups:
                grp.pool = torch.zeros((len(grp.slots), num_pages, 2, grp.need.num_kv_heads, page_size, grp.need.head_dim),
                                       dtype=dtype, device=self.device)
            for key, need in state_needs.items():
                shape, state_dtype = state_shape_dtype(need)
                self.states.tensors[key] = torch.zeros((max_requests, *shape), dtype=state_dtype, device=self.device)
        self.has_state = bool(state_needs)

    # ---- capacity
    @property
    def capacity_tokens(self) -> int:
        """The longest request the pool can hold alone."""
        return min(self.num_pages * self.page_size, self.max_model_len)

    @property
    def num_free_pages(self) -> int:
        return min((g.allocator.num_free for g in self.groups), default=self.num_pages)

    def pages_needed(self, req: Hashable, n_tokens: int) -> list[int]:
        c = self.computed.get(req, 0)
        return [g.pages_needed(req, c, n_tokens) for g in self.groups]

    def can_ensure(self, req: Hashable, n_tokens: int) -> bool:
        if n_tokens > self.max_model_len:
            return False
        if self.has_state and req not in self.states.owner and not self.states.num_free:
            return False
        return all(n <= g.allocator.num_free for n, g in zip(self.pages_needed(req, n_tokens), self.groups))

    # ---- a request's life
    def ensure(self, req: Hashable, n_tokens: int) -> None:
        """Back positions [computed, n_tokens) of `req` with pages in every group (all or nothing)."""
        if n_tokens > self.max_model_len:
            raise ValueError(f"{n_tokens} tokens exceed max_model_len {self.max_model_len}")
        # the common case of a decode step: the request's last page still has room in every group (and it has its state)
        if req in self.computed and (not self.has_state or req in self.states.owner):
            for g in self.groups:
                if g.lens.get(req, 0) * g.page_size < n_tokens:
                    break
            else:
                return
        if not self.can_ensure(req, n_tokens):
            raise OutOfPages(f"request {req!r} needs {self.pages_needed(req, n_tokens)} more pages per group for "
                             f"{n_tokens} tokens; free: {[g.allocator.num_free for g in self.groups]}")
        c = self.computed.setdefault(req, 0)
        for g in self.groups:
            g.ensure(req, c, n_tokens)
        if self.has_state:
            self.states.acquire(req)

    def commit(self, req: Hashable, n_computed: int) -> None:
        """Positions [0, n_computed) of `req` are in the cache: window groups give back what lies before the window."""
        if req not in self.computed:
            raise KeyError(f"request {req!r} holds nothing")
        self.computed[req] = n_computed
        for g in self.groups:
            g.release_before(req, n_computed)

    def free(self, req: Hashable) -> None:
        for g in self.groups:
            g.free(req)
        self.computed.pop(req, None)
        self.states.release(req)

    def reclaim(self, req: Hashable, n_tokens: int, victims) -> list[Hashable]:
        """Frees requests out of `victims` (an iterable of request ids, taken in the order given) until `req` can be
        backed for n_tokens or none is left. Returns the ids that were freed; whether it was enough is what
        `can_ensure` says afterwards. A victim that holds nothing is passed over."""
        freed = []
        for v in victims:
            if self.can_ensure(req, n_tokens):
                break
            if v == req or v not in self.computed:
                continue
            self.free(v)
            freed.append(v)
        return freed

    def reset(self) -> None:
        for req in list(self.computed):
            self.free(req)

    def holds(self, req: Hashable) -> bool:
        return req in self.computed

    def live_requests(self) -> list[Hashable]:
        return list(self.computed)

    # ---- views for the step function
    def table(self, group: int, req: Hashable) -> list[int]:
        g = self.groups[group]
        return g.rows[req][: g.lens[req]].tolist() if req in g.rows else []

    def table_row(self, group: int, req: Hashable) -> tuple[np.ndarray | None, int]:
        """(int32 row of page ids, entries in use) without copying; (None, 0) for a request that holds nothing."""
        g = self.groups[group]
        return g.rows.get(req), g.lens.get(req, 0)

    def state_slot(self, req: Hashable) -> int:
        return self.states.owner.get(req, -1)

    def check(self) -> None:
        """Invariants: allocators consistent, and every held page is in exactly one table of its group."""
        for g in self.groups:
            g.allocator.check()
            seen: set[int] = set()
            for req, t in g.tables.items():
                assert all(p >= 0 for p in t[g.first_live_page(self.computed.get(req, 0)):]), f"{req!r} lacks a live page"
                for p in t:
                    if p >= 0:
                        assert p not in seen, f"page {p} is in two block tables"
                        seen.add(p)
            assert len(seen) == g.num_pages - g.allocator.num_free, \
                f"{g.num_pages - g.allocator.num_free} pages held, {len(seen)} in tables"
        assert len(set(self.states.owner.values())) == len(self.states.owner), "a state slot has two owners"
        assert len(self.states.owner) + self.states.num_free == self.states.num_slots, "a state slot is lost"
