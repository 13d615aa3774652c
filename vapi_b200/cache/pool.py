"""Page and slot allocators (host side, no tensors).

``PagePool`` is the allocator of the reference's block pool without its content index
(crates/vapi-cache/src/pool.rs:80-247): a free list, an owner count per page, and a
watermark of pages that admission may not touch (``can_allocate``) while running requests
still may (``allocate``).  Freed pages go to the front of the list and are handed out
again first, so a small pool reuses pages quickly.
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Iterable, List


class OutOfPages(RuntimeError):
    pass


class OutOfSlots(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int, watermark_pages: int = 0):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self.watermark = max(0, min(int(watermark_pages), self.num_pages - 1))
        self._free: Deque[int] = deque(range(self.num_pages))
        self._held = [False] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def can_allocate(self, n: int) -> bool:
        """Whether admission may take ``n`` pages and still leave the watermark."""
        return self.num_free >= n + self.watermark

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        p = self._free.popleft()
        self._held[p] = True
        return p

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise ValueError(f"page {page} is outside the pool")
        if not self._held[page]:
            raise ValueError(f"page {page} is freed twice")
        self._held[page] = False
        self._free.appendleft(page)

    def free_all(self, pages: Iterable[int]) -> None:
        for p in pages:
            self.free(p)

    def held_pages(self) -> List[int]:
        return [i for i, h in enumerate(self._held) if h]

    def check_invariants(self) -> None:
        free = list(self._free)
        assert len(set(free)) == len(free), "a page is on the free list twice"
        for p in free:
            assert not self._held[p], f"page {p} is free and held"
        assert len(free) + sum(self._held) == self.num_pages, "a page is lost"


class SlotPool:
    """Slots for per-request state of fixed size."""

    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError("a slot pool needs at least one slot")
        self.num_slots = int(num_slots)
        self._free: Deque[int] = deque(range(self.num_slots))
        self._held = [False] * self.num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self) -> int:
        if not self._free:
            raise OutOfSlots("no free state slot")
        s = self._free.popleft()
        self._held[s] = True
        return s

    def release(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots:
            raise ValueError(f"slot {slot} is outside the pool")
        if not self._held[slot]:
            raise ValueError(f"slot {slot} is released twice")
        self._held[slot] = False
        self._free.appendleft(slot)

    def check_invariants(self) -> None:
        free = list(self._free)
        assert len(set(free)) == len(free), "a slot is on the free list twice"
        for s in free:
            assert not self._held[s]
        assert len(free) + sum(self._held) == self.num_slots, "a slot is lost"
