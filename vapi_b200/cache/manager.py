"""The cache manager: paged keys/values per group of layers, and state slots per request.

Call sites of the model's run order that own a cache are grouped by what they need:

* a **paged group** per distinct :class:`~vapi_b200.parts.base.PagedSpec` (the buffers a mixer
  keeps per token, and its window).  Each group has pages of its own: one pool, one device
  tensor ``[sites, pages, page_size * elements per token]`` and one block table per request.
  Inside a page the spec's buffers follow one another, each as ``[rows, page_size, width]``, so
  keys and values of ``n_kv`` heads lie as ``[2, n_kv, page_size, head_dim]``; the manager
  itself only knows sizes.  A group with a window gives pages back as soon as the window has
  passed them.
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

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import PagedSpec, StateSpec
from .. import hostlib
from .pool import OutOfSlots, PagePool, SlotPool


@dataclass
class PagedGroup:
    spec: PagedSpec
    sites: List[int]
    pool: PagePool
    tensor: torch.Tensor            # [sites, pages, page_size * elements per token]

    def bytes_per_token(self) -> int:
        return len(self.sites) * self.spec.elems_per_token() * self.tensor.element_size()


@dataclass
class StateGroup:
    spec: StateSpec
    sites: List[int]
    tensor: torch.Tensor            # [slots + 1, sites, *shape]


class RequestCache:
    """What one live request holds.  The books themselves (block tables per paged group, the
    state slot, the count of computed positions) live in the host runtime; this object is the
    request's handle to them."""

    __slots__ = ("request_id", "handle", "slot", "closed", "_mgr", "_final_tokens")

    def __init__(self, mgr: "CacheManager", request_id, handle: int, slot: int):
        self._mgr, self.request_id, self.handle, self.slot = mgr, request_id, handle, slot
        self.closed = False
        self._final_tokens = 0

    @property
    def num_tokens(self) -> int:
        """Positions computed so far."""
        if self.closed:
            return self._final_tokens
        return self._mgr._lib.vh_num_tokens(self._mgr._h, self.handle)

    @property
    def tables(self) -> List[List[int]]:
        """Per paged group: page id per logical page, -1 once the window released it."""
        if self.closed:
            return [[] for _ in self._mgr.paged]
        return [self._mgr._table(self.handle, g) for g in range(len(self._mgr.paged))]

    @property
    def first_live(self) -> List[int]:
        """Per paged group: first logical page still held."""
        if self.closed:
            return [0 for _ in self._mgr.paged]
        return [self._mgr._lib.vh_first_live(self._mgr._h, self.handle, g) for g in range(len(self._mgr.paged))]


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
        if self.max_requests <= 0:
            raise ValueError("a slot pool needs at least one slot")
        sizes = []
        for spec in by_paged:
            n_pages = int((pages_per_group or {}).get(spec, num_pages))
            if n_pages <= 0:
                raise ValueError("the cache needs at least one page per group")
            wm = int(-(-n_pages * watermark // 1)) if watermark > 0 else 0
            sizes.append((n_pages, wm, max(int(spec.window), 0)))
        self._lib = hostlib.lib()
        cols = [hostlib.i32([z[k] for z in sizes] or [0]) for k in range(3)]
        self._h = self._lib.vh_cache_new(len(sizes), self.page_size, cols[0].ctypes.data, cols[1].ctypes.data,
                                         cols[2].ctypes.data, self.max_requests)
        if not self._h:
            raise ValueError(hostlib.last_error())
        for gi, (spec, ss) in enumerate(by_paged.items()):
            t = torch.empty((len(ss), sizes[gi][0], self.page_size * spec.elems_per_token()),
                            dtype=dtype, device=self.device)
            pool = PagePool(borrowed=self._lib.vh_cache_group_pool(self._h, gi), owner=self)
            self.paged.append(PagedGroup(spec, list(ss), pool, t))
            for j, s in enumerate(ss):
                self._site[s] = ("paged", gi, j)
        self.slots = SlotPool(borrowed=self._lib.vh_cache_slot_pool(self._h), owner=self)
        for spec, ss in by_state.items():
            t = torch.empty((self.max_requests + 1, len(ss)) + tuple(spec.shape),
                            dtype=spec.dtype or dtype, device=self.device)
            gi = len(self.state)
            self.state.append(StateGroup(spec, list(ss), t))
            for j, s in enumerate(ss):
                self._site[s] = ("state", gi, j)
        self._live: Dict[object, RequestCache] = {}
        self._scratch = np.empty(64, dtype=np.int32)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.vh_cache_delete(h)

    @property
    def native(self) -> int:
        """The host runtime's handle of this cache's books (for the packer and the scheduler)."""
        return self._h

    def _table(self, handle: int, group: int) -> List[int]:
        n = self._lib.vh_table(self._h, handle, group, self._scratch.ctypes.data, self._scratch.size)
        if n > self._scratch.size:
            self._scratch = np.empty(2 * n, dtype=np.int32)
            n = self._lib.vh_table(self._h, handle, group, self._scratch.ctypes.data, self._scratch.size)
        return self._scratch[:n].tolist()

    # ---- what the model sees -------------------------------------------------------
    @property
    def scratch_slot(self) -> int:
        """A slot no request ever owns; padding rows of a captured step point here."""
        return self.max_requests

    def site_kind(self, site: int) -> Tuple[str, int]:
        kind, gi, _ = self._site.get(site, ("none", -1, -1))
        return kind, gi

    def site_tensor(self, site: int) -> Optional[torch.Tensor]:
        """This call site's part of the cache: its pages, flat [pages, page_size * elements per
        token], or its states [slots+1, *shape]."""
        if site not in self._site:
            return None
        kind, gi, j = self._site[site]
        if kind == "paged":
            return self.paged[gi].tensor[j]
        return self.state[gi].tensor[:, j]

    def site_buffers(self, site: int) -> Optional[Dict[str, torch.Tensor]]:
        """A paged call site's pages seen buffer by buffer: name -> [pages, rows, page_size, width]
        (views of the same memory; the stride between pages is the whole page)."""
        if site not in self._site or self._site[site][0] != "paged":
            return None
        _, gi, j = self._site[site]
        spec, flat = self.paged[gi].spec, self.paged[gi].tensor[j]
        out, off = {}, 0
        for b in spec.buffers:
            out[b.name] = flat.as_strided((flat.shape[0], b.rows, self.page_size, b.width),
                                          (flat.stride(0), self.page_size * b.width, b.width, 1), flat.storage_offset() + off)
            off += b.rows * self.page_size * b.width
        return out

    def site_spec(self, site: int):
        """The spec of the group that the call site's cache belongs to."""
        if site not in self._site:
            return None
        kind, gi, _ = self._site[site]
        return self.paged[gi].spec if kind == "paged" else self.state[gi].spec

    def set_aside_pages(self) -> Optional[List[int]]:
        """Take one page per paged group out of circulation (for the padding rows of a
        fixed-shape decode step, like the reference's reserved blocks,
        crates/vapi-backend-candle/src/backend.rs:426-438).  None if a group has no free page."""
        out = np.zeros(max(len(self.paged), 1), dtype=np.int32)
        if not self._lib.vh_set_aside(self._h, out.ctypes.data):
            return None
        return out[:len(self.paged)].tolist()

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
        h = self._lib.vh_open(self._h)
        if h < 0:
            raise OutOfSlots("no free state slot")
        rc = RequestCache(self, request_id, h, self._lib.vh_slot(self._h, h))
        self._live[request_id] = rc
        return rc

    def adopt(self, request_id, handle: int) -> RequestCache:
        """The Python face of a request that the host runtime's scheduler opened itself."""
        rc = RequestCache(self, request_id, handle, self._lib.vh_slot(self._h, handle))
        self._live[request_id] = rc
        return rc

    def forget(self, rc: RequestCache) -> None:
        """The host runtime's scheduler has closed this request; only the Python face remains."""
        if not rc.closed:
            rc._final_tokens = 0
            rc.closed = True
        self._live.pop(rc.request_id, None)

    def live(self, request_id) -> Optional[RequestCache]:
        return self._live.get(request_id)

    def pages_needed(self, rc: Optional[RequestCache], total: int) -> List[int]:
        """New pages each group would need so that positions < total are covered."""
        have = [len(t) for t in rc.tables] if rc is not None else [0] * len(self.paged)
        return [max(0, self.pages_for(total) - h) for h in have]

    def can_admit(self, total: int) -> bool:
        """Whether a new request of ``total`` tokens fits while leaving the watermark."""
        return bool(self._lib.vh_can_admit(self._h, int(total)))

    def reserve(self, rc: RequestCache, total: int, guarded: bool = False) -> bool:
        """Make sure every paged group covers positions < ``total``.  All or nothing: on
        failure the request holds what it held before.  ``guarded`` respects the watermark
        (admission); running requests reserve unguarded, as in the reference
        (crates/vapi-engine/src/scheduler.rs:464-507)."""
        assert not rc.closed
        r = self._lib.vh_reserve(self._h, rc.handle, int(total), 1 if guarded else 0)
        if r < 0:
            raise ValueError(hostlib.last_error())
        return r == 1

    def commit(self, rc: RequestCache, total: int) -> None:
        """The request has computed positions < ``total``.  A windowed group gives back
        every page all of whose positions are out of reach of any later query: the next
        query sits at a position >= total and sees keys > total - window."""
        assert not rc.closed
        self._lib.vh_commit(self._h, rc.handle, int(total))

    def close(self, rc: RequestCache) -> None:
        if rc.closed:
            raise ValueError(f"request {rc.request_id!r} is closed twice")
        rc._final_tokens = rc.num_tokens
        if self._lib.vh_close(self._h, rc.handle) != 0:
            raise ValueError(f"request {rc.request_id!r}: {hostlib.last_error()}")
        rc.closed = True
        self._live.pop(rc.request_id, None)

    def slot_of(self, rc: RequestCache, group: int, position: int) -> int:
        page = self._table(rc.handle, group)[position // self.page_size]
        if page < 0:
            raise ValueError(f"position {position} lies in a page the window has released")
        return page * self.page_size + position % self.page_size

    # ---- checks ----------------------------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, held twice or freed twice; the same for slots."""
        if self._lib.vh_cache_check(self._h) != 0:
            raise AssertionError(hostlib.last_error())
