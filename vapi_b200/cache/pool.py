"""Page and slot allocators (host side, no tensors).

The books are kept by the host runtime in C++ (``csrc/host.cpp``); these classes are its
Python face.  ``PagePool`` is the allocator of the reference's block pool without its
content index (crates/vapi-cache/src/pool.rs:80-247): a free list, a held flag per page, and a
watermark of pages that admission may not touch (``can_allocate``) while running requests
still may (``allocate``).  Freed pages go to the front of the list and are handed out
again first, so a small pool reuses pages quickly.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import numpy as np

from .. import hostlib


class OutOfPages(RuntimeError):
    pass


class OutOfSlots(RuntimeError):
    pass


class _Pool:
    _what = "id"

    def __init__(self, count: int, watermark: int = 0, *, borrowed: Optional[int] = None, owner=None):
        self._lib = hostlib.lib()
        if borrowed is not None:
            self._h, self._own, self._owner = borrowed, False, owner     # lives inside a cache's books
        else:
            if count <= 0:
                raise ValueError(f"a {self._what} pool needs at least one {self._what}")
            self._h, self._own, self._owner = self._lib.vh_pool_new(int(count), int(watermark)), True, None
        self._n = self._lib.vh_pool_size(self._h)

    def __del__(self):
        if getattr(self, "_own", False) and self._h:
            self._lib.vh_pool_delete(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return self._lib.vh_pool_num_free(self._h)

    def _take(self) -> int:
        return self._lib.vh_pool_allocate(self._h)

    def _give(self, i: int, twice: str) -> None:
        rc = self._lib.vh_pool_release(self._h, int(i))
        if rc == -1:
            raise ValueError(f"{self._what} {i} is outside the pool")
        if rc == -2:
            raise ValueError(f"{self._what} {i} is {twice} twice")

    def held(self) -> List[int]:
        out = np.empty(self._n, dtype=np.int32)
        k = self._lib.vh_pool_held(self._h, out.ctypes.data, self._n)
        return out[:k].tolist()

    def check_invariants(self) -> None:
        if self._lib.vh_pool_check(self._h) != 0:
            raise AssertionError(hostlib.last_error())


class PagePool(_Pool):
    _what = "page"

    def __init__(self, num_pages: int = 0, watermark_pages: int = 0, **kw):
        super().__init__(num_pages, watermark_pages, **kw)

    @property
    def num_pages(self) -> int:
        return self._n

    @property
    def watermark(self) -> int:
        return self._lib.vh_pool_watermark(self._h)

    def can_allocate(self, n: int) -> bool:
        """Whether admission may take ``n`` pages and still leave the watermark."""
        return bool(self._lib.vh_pool_can_allocate(self._h, int(n)))

    def allocate(self) -> int:
        p = self._take()
        if p < 0:
            raise OutOfPages("no free page")
        return p

    def free(self, page: int) -> None:
        self._give(page, "freed")

    def free_all(self, pages: Iterable[int]) -> None:
        for p in pages:
            self.free(p)

    def held_pages(self) -> List[int]:
        return self.held()


class SlotPool(_Pool):
    """Slots for per-request state of fixed size."""
    _what = "slot"

    def __init__(self, num_slots: int = 0, **kw):
        super().__init__(num_slots, 0, **kw)

    @property
    def num_slots(self) -> int:
        return self._n

    def acquire(self) -> int:
        s = self._take()
        if s < 0:
            raise OutOfSlots("no free state slot")
        return s

    def release(self, slot: int) -> None:
        self._give(slot, "released")
