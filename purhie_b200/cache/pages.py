"""Page bookkeeping on the host: a free list with reference counts, and fixed-size state slots.

Nothing here touches a device, so the bookkeeping is tested without one.  The reference keeps one
cache per sequence, made of blocks of 256 positions that are registered as positions reach them and
are never given back before the sequence is freed (src/kv_cache.cpp:133-226, 242-260;
src/inference.cpp:1784-1802); a block can be shared with a store and made private again
(src/kv_cache.cpp:266-347), which is what the reference counts here are kept for.
"""
from __future__ import annotations

from typing import Iterable, List


class OutOfPages(RuntimeError):
    """The pool has fewer free pages than were asked for.  Nothing was taken."""


class OutOfSlots(RuntimeError):
    """Every per-request state slot is in use."""


class PageAllocator:
    """``num_pages`` pages numbered from 0.  A page is free or held with a reference count >= 1."""

    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self.num_pages = num_pages
        # A stack: the page freed last is handed out first, so that reuse happens early.
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._ref: List[int] = [0] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} of {self.num_pages} free")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._ref[p] = 1
        return pages

    def share(self, page: int) -> None:
        if self._ref[page] < 1:
            raise ValueError(f"page {page} is free and cannot be shared")
        self._ref[page] += 1

    def refcount(self, page: int) -> int:
        return self._ref[page]

    def free(self, pages: Iterable[int]) -> List[int]:
        """Drop one reference of each page; returns the pages that became free."""
        released = []
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is outside the pool of {self.num_pages}")
            if self._ref[p] < 1:
                raise ValueError(f"page {p} freed twice")
            self._ref[p] -= 1
            if self._ref[p] == 0:
                self._free.append(p)
                released.append(p)
        return released

    def check(self) -> None:
        """Raise AssertionError unless every page is exactly free or held."""
        free = set(self._free)
        assert len(free) == len(self._free), "a page is on the free list twice"
        for p in range(self.num_pages):
            assert (self._ref[p] == 0) == (p in free), f"page {p}: refcount {self._ref[p]}, on free list: {p in free}"


class SlotAllocator:
    """``num_slots`` slots for per-request state of fixed size (one slot per live request)."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free: List[int] = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.num_slots} state slots are in use")
        s = self._free.pop()
        self._held[s] = True
        return s

    def free(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise ValueError(f"slot {slot} is not held")
        self._held[slot] = False
        self._free.append(slot)

    def check(self) -> None:
        free = set(self._free)
        assert len(free) == len(self._free), "a slot is on the free list twice"
        for s in range(self.num_slots):
            assert self._held[s] != (s in free), f"slot {s} is both held and free, or neither"
