"""Page and slot allocators: plain host bookkeeping, no device memory.

`PageAllocator` hands out page ids from a LIFO free list, so a page that was just given back is the next one handed
out (the reference's BlockAllocator does the same: fusezap/serve/kv_cache.py:43-65). It raises `OutOfPages` when short
and refuses to free a page that is not held, so no page can be lost, held twice or freed twice without an error.
"""
from __future__ import annotations


class OutOfPages(MemoryError):
    pass


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"num_pages must be positive, got {num_pages}")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))   # pop() hands out page 0 first
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, n: int) -> list[int]:
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} of {self.num_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def free(self, pages: list[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages or not self._held[p]:
                raise AssertionError(f"page {p} is not held (freed twice, or never allocated)")
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """Every page is either free or held, never both, never neither."""
        free = set(self._free)
        assert len(free) == len(self._free), "a page is on the free list twice"
        for p in range(self.num_pages):
            assert (p in free) != self._held[p], f"page {p}: free={p in free} held={self._held[p]}"
