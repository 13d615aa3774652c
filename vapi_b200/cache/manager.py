"""The cache manager: paged keys/values per group of layers, and state slots per request.

Call sites of the model's run order that own a cache are grouped by what they need:

* a **paged group** per distinct :class:`~vapi_b200.parts.base.PagedSpec` (kv heads, head
  size, window).  Each group has pages of its own: one pool, one device tensor
  ``[sites, pages, 2, n_kv, page_size, head_dim]`` and one block table per request.  A group
  with a window gives pages back as soon as the window has passed them.
* a **state group** per distinct :class:`~vapi_b200.parts.base.StateSpec`: one device tensor
  ``[slots + 1, sites, *shape]``.  All state groups share one slot pool, so a request holds a
  single slot index that is valid in every state tensor.  The extra last slot is a scratch
  slot that padding rows of a captured decode step write to.  Slots exist even for a model
  without any stateful mixer (the pool is then only bookkeeping).

The reference keeps conv rows per token in the same paged block space as K/V
(crates/vapi-backend-candle/src/cache.rs:22-45, models/lfm2.rs:145-160); here the
fixed-size state has slots of its own and the pages hold attention K/V only.

A request's life: ``open`` (takes a slot) -> ``reserve(total)`` before each step (pages for
positions < total in every paged group; False when pages run out, nothing kept) ->
``commit(total)`` after the step (windowed groups release what fell behind) -> ``close``
(everything goes back).  Memory is never cleared on reuse.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheView, PagedSpec, StateSpec
from .pool import OutOfPages, OutOfSlots, PagePool, SlotPool


@dataclass
class PagedGroup:
    spec: PagedSpec
    sites: List[int]
    pool: PagePool
    tensor: torch.Tensor            # [sites, pages, 2, n_kv, page_size, head_dim]

    def bytes_per_token(self) -> int:
        return len(self.sites) * self.spec.elems_per_token() * self.tensor.element_size()


@dataclass
class StateGroup:
    spec: StateSpec
    sites: List[int]
    tensor: torch.Tensor            # [slots + 1, sites, *shape]


@dataclass
class RequestCache:
    """What one live request holds."""

    request_id: object
    slot: int
    tables: List[List[int]]         # per paged group: page id per logical page, -1 once released
    first_live: List[int]           # per paged group: first logical page still held
    num_tokens: int = 0             # positions computed so far
    closed: bool = False
    # per paged group, the same table as an int32 array for the step packer (released pages
    # read 0, a valid id no kernel follows); grown in place, `tables` stays the truth
    tables_np: List[np.ndarray] = field(default_factory=list)

    def table_row(self, group: int, width: int) -> np.ndarray:
        n = min(width, len(self.tables[group]))
        return self.tables_np[group][:n]


class CacheManager:
    def __init__(self, sites: Sequence[Tuple[int, object]], *, page_size: int, num_pages: int,
                 max_requests: int, dtype: torch.dtype, device, watermark: float = 0.0,
                 pages_per_group: Optional[Dict[PagedSpec, int]] = None):
        if page_size <= 0 or page_size % 16:
            raise ValueError(f"page size {page_size} must be a positive multiple of 16")
        self.page_size, self.dtype, self.device = int(page_size), dtype, torch.device(device)
        self.max_requests = int(max_requests)
        self.paged: List[PagedGroup] = []
        self.state: List[StateGroup] = []
        self._site: Dict[int, Tuple[str, int, int]] = {}    # site -> (kind, group index, index in group)
        by_paged: Dict[PagedSpec, List[int]] = {}
        by_state: Dict[StateSpec, List[int]] = {}
        for site, spec in sites:
            if isinstance(spec, PagedSpec):
                by_paged.setdefault(spec, []).append(site)
            elif isinstance(spec, StateSpec):
                by_state.setdefault(spec, []).append(site)
            else:
                raise TypeError(f"run order entry {site}: unknown cache spec {spec!r}")
        for spec, ss in by_paged.items():
            n_pages = int((pages_per_group or {}).get(spec, num_pages))
            if n_pages <= 0:
                raise ValueError("the cache needs at least one page per group")
            wm = int(-(-n_pages * watermark // 1)) if watermark > 0 else 0
            t = torch.empty((len(ss), n_pages, 2, spec.n_kv, self.page_size, spec.head_dim),
                            dtype=dtype, device=self.device)
            gi = len(self.paged)
            self.paged.append(PagedGroup(spec, list(ss), PagePool(n_pages, wm), t))
            for j, s in enumerate(ss):
                self._site[s] = ("paged", gi, j)
        self.slots = SlotPool(self.max_requests)
        for spec, ss in by_state.items():
            t = torch.empty((self.max_requests + 1, len(ss)) + tuple(spec.shape),
                            dtype=spec.dtype or dtype, device=self.device)
            gi = len(self.state)
            self.state.append(StateGroup(spec, list(ss), t))
            for j, s in enumerate(ss):
                self._site[s] = ("state", gi, j)
        self._live: Dict[object, RequestCache] = {}
        self._set_aside: List[List[int]] = [[] for _ in self.paged]

    # ---- what the model sees -------------------------------------------------------
    @property
    def scratch_slot(self) -> int:
        """A slot no request ever owns; padding rows of a captured step point here."""
        return self.max_requests

    def site_kind(self, site: int) -> Tuple[str, int]:
        kind, gi, _ = self._site.get(site, ("none", -1, -1))
        return kind, gi

    def site_tensor(self, site: int) -> Optional[torch.Tensor]:
        """This call site's part of the cache: [pages, 2, n_kv, page, d] or [slots+1, *shape]."""
        if site not in self._site:
            return None
        kind, gi, j = self._site[site]
        if kind == "paged":
            return self.paged[gi].tensor[j]
        return self.state[gi].tensor[:, j]

    def set_aside_pages(self) -> Optional[List[int]]:
        """Take one page per paged group out of circulation (for the padding rows of a
        fixed-shape decode step, like the reference's reserved blocks,
        crates/vapi-backend-candle/src/backend.rs:426-438).  None if a group has no free page."""
        if any(g.pool.num_free == 0 for g in self.paged):
            return None
        pages = []
        for gi, g in enumerate(self.paged):
            p = g.pool.allocate()
            self._set_aside[gi].append(p)
            pages.append(p)
        return pages

    # ---- sizing -----------------------------------------------------------------------
    def pages_for(self, tokens: int) -> int:
        return -(-int(tokens) // self.page_size)

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.paged)

    def state_bytes_per_request(self) -> int:
        return sum(g.tensor[0].numel() * g.tensor.element_size() for g in self.state)

    # ---- a request's life ----------------------------------------------------------
    def open(self, request_id) -> RequestCache:
        if request_id in self._live:
            raise ValueError(f"request {request_id!r} is already live")
        slot = self.slots.acquire()
        rc = RequestCache(request_id, slot, [[] for _ in self.paged], [0 for _ in self.paged],
                          tables_np=[np.zeros(16, dtype=np.int32) for _ in self.paged])
        self._live[request_id] = rc
        return rc

    def live(self, request_id) -> Optional[RequestCache]:
        return self._live.get(request_id)

    def pages_needed(self, rc: Optional[RequestCache], total: int) -> List[int]:
        """New pages each group would need so that positions < total are covered."""
        out = []
        for gi, g in enumerate(self.paged):
            have = len(rc.tables[gi]) if rc is not None else 0
            out.append(max(0, self.pages_for(total) - have))
        return out

    def can_admit(self, total: int) -> bool:
        """Whether a new request of ``total`` tokens fits while leaving the watermark."""
        if self.slots.num_free == 0:
            return False
        return all(g.pool.can_allocate(n) for g, n in zip(self.paged, self.pages_needed(None, total)))

    def reserve(self, rc: RequestCache, total: int, guarded: bool = False) -> bool:
        """Make sure every paged group covers positions < ``total``.  All or nothing: on
        failure the request holds what it held before.  ``guarded`` respects the watermark
        (admission); running requests reserve unguarded, as in the reference
        (crates/vapi-engine/src/scheduler.rs:464-507)."""
        assert not rc.closed
        need = self.pages_needed(rc, total)
        for g, n in zip(self.paged, need):
            if (guarded and not g.pool.can_allocate(n)) or g.pool.num_free < n:
                return False
        for gi, (g, n) in enumerate(zip(self.paged, need)):
            for _ in range(n):
                page = g.pool.allocate()
                k = len(rc.tables[gi])
                if k >= rc.tables_np[gi].size:
                    grown = np.zeros(max(2 * rc.tables_np[gi].size, k + 1), dtype=np.int32)
                    grown[:k] = rc.tables_np[gi][:k]
                    rc.tables_np[gi] = grown
                rc.tables_np[gi][k] = page
                rc.tables[gi].append(page)
        return True

    def commit(self, rc: RequestCache, total: int) -> None:
        """The request has computed positions < ``total``.  A windowed group gives back
        every page all of whose positions are out of reach of any later query: the next
        query sits at a position >= total and sees keys > total - window."""
        assert not rc.closed
        rc.num_tokens = int(total)
        for gi, g in enumerate(self.paged):
            w = g.spec.window
            if w <= 0:
                continue
            dead_upto = total - w          # keys <= dead_upto are never read again
            while True:
                pi = rc.first_live[gi]
                if pi >= len(rc.tables[gi]) or (pi + 1) * self.page_size - 1 > dead_upto:
                    break
                g.pool.free(rc.tables[gi][pi])
                rc.tables[gi][pi] = -1
                rc.tables_np[gi][pi] = 0
                rc.first_live[gi] = pi + 1

    def close(self, rc: RequestCache) -> None:
        if rc.closed:
            raise ValueError(f"request {rc.request_id!r} is closed twice")
        for gi, g in enumerate(self.paged):
            g.pool.free_all(p for p in rc.tables[gi] if p >= 0)
            rc.tables[gi] = []
        self.slots.release(rc.slot)
        rc.closed = True
        self._live.pop(rc.request_id, None)

    def slot_of(self, rc: RequestCache, group: int, position: int) -> int:
        page = rc.tables[group][position // self.page_size]
        if page < 0:
            raise ValueError(f"position {position} lies in a page the window has released")
        return page * self.page_size + position % self.page_size

    # ---- checks ----------------------------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, held twice or freed twice; the same for slots."""
        for gi, g in enumerate(self.paged):
            g.pool.check_invariants()
            held = sorted([p for rc in self._live.values() for p in rc.tables[gi] if p >= 0] + self._set_aside[gi])
            assert len(set(held)) == len(held), "a page is held by two requests"
            assert held == g.pool.held_pages(), "pool and requests disagree about held pages"
        self.slots.check_invariants()
        slots = [rc.slot for rc in self._live.values()]
        assert len(set(slots)) == len(slots), "a slot is held by two requests"
        assert self.slots.num_free + len(slots) == self.slots.num_slots, "a slot is lost"
