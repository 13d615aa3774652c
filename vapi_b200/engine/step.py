"""A step's batch on the host and its metadata on the device.

A step is a list of entries, one per request that takes part: the request's next tokens
(a portion of its prompt, or one decoded token) and the places among them whose logits are
wanted.  It plays the part of the reference's ``ForwardBatch``
(crates/vapi-engine/src/backend.rs:47-75) with two differences: slot mappings and block
tables exist once per paged cache group, and each sequence also names its state slot.

All index data of a step is packed into one int32 buffer and goes to the device in a
single copy; the tensors of :class:`StepContext` are views into it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import hostlib
from ..cache.manager import CacheManager, RequestCache


class StepError(ValueError):
    """A batch that breaks an invariant of the step function."""


@dataclass
class StepEntry:
    cache: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()

    @property
    def start(self) -> int:
        return self.cache.num_tokens


@dataclass
class GroupMeta:
    """What a step holds for one paged cache group.  ``splits`` and ``max_k`` are set for steps
    of a fixed shape (captured decode steps), where they cannot follow the batch: into how many
    slices the group's mixers cut a sequence's keys, and the most keys a sequence of the group can
    have.  None leaves the choice to the mixer and to the step's own ``max_k``."""
    slot_mapping: torch.Tensor      # [n] int32: page * page_size + offset of each token
    block_table: torch.Tensor       # [S, width] int32
    splits: Optional[int] = None
    max_k: Optional[int] = None


@dataclass
class StepContext:
    n: int
    num_seqs: int
    num_rows: int                   # rows of logits wanted
    max_q: int
    max_k: int
    tokens: torch.Tensor
    positions: torch.Tensor
    tok_seq: torch.Tensor
    cu_q: torch.Tensor
    seqlens_k: torch.Tensor
    state_slots: torch.Tensor
    logits_rows: Optional[torch.Tensor]
    groups: List[GroupMeta]
    dtype: torch.dtype
    status: Optional[torch.Tensor] = None
    attention_splits: Optional[int] = None
    token_src: Optional[torch.Tensor] = None   # [n] int32: >= 0 where a token is a row of the last sampled output
    unknown_tokens: bool = False    # some token_src is >= 0: fetch those tokens on the device first
    rows_identity: bool = False     # the wanted rows are exactly rows 0 .. n-1 in order
    fused: bool = False             # a step of few rows: norms and adds ride on the matrix products
    pos: Dict[str, Any] = field(default_factory=dict)
    extras: Dict[str, Any] = field(default_factory=dict)


def validate_step(entries: Sequence[StepEntry], cache: CacheManager, vocab: int, max_positions: int) -> None:
    """The invariants the reference checks on every batch
    (crates/vapi-engine/src/backend.rs:96-204), in this engine's terms."""
    if not entries:
        raise StepError("a step needs at least one entry")
    seen = set()
    for e in entries:
        rc = e.cache
        if rc.closed:
            raise StepError(f"request {rc.request_id!r} has ended")
        if id(rc) in seen:
            raise StepError(f"request {rc.request_id!r} appears twice in one step")
        seen.add(id(rc))
        q = len(e.tokens)
        if q == 0:
            raise StepError(f"request {rc.request_id!r} brings no tokens")
        if e.start + q > max_positions:
            raise StepError(f"request {rc.request_id!r} would pass position {max_positions}")
        for t in e.tokens:
            if not 0 <= int(t) < vocab:
                raise StepError(f"request {rc.request_id!r}: token {t} is outside the vocabulary of {vocab}")
        for w in e.want:
            if not 0 <= int(w) < q:
                raise StepError(f"request {rc.request_id!r}: wanted place {w} is outside its {q} tokens")
        need = cache.pages_for(e.start + q)
        for gi, table in enumerate(rc.tables):
            if len(table) < need:
                raise StepError(f"request {rc.request_id!r}: {len(table)} pages do not cover {e.start + q} tokens")
            lo = rc.first_live[gi]
            first_needed = max(0, e.start - max(cache.paged[gi].spec.window, 0) + 1) // cache.page_size \
                if cache.paged[gi].spec.window > 0 else 0
            if lo > first_needed:
                raise StepError(f"request {rc.request_id!r}: a page inside the window was released")
            live = [p for p in table[lo:need]]
            if any(p < 0 or p >= cache.paged[gi].pool.num_pages for p in live):
                raise StepError(f"request {rc.request_id!r}: page id out of range")
        if not 0 <= rc.slot < cache.max_requests:
            raise StepError(f"request {rc.request_id!r}: state slot out of range")


def _round_up(x: int, m: int) -> int:
    return -(-x // m) * m


class StepPacker:
    """Packs a step's index data and ships it to the device in one copy.

    The layout depends only on (token capacity, sequence capacity, table width), so a
    captured decode step of a given bucket always finds its inputs at the same addresses.
    Pinned staging buffers are used in rotation; an event guards each against being
    overwritten while its copy is still in flight.
    """

    def __init__(self, cache: CacheManager, device, max_tokens: int, max_seqs: int, max_table_width: int,
                 ring: int = 3):
        self.cache, self.device = cache, torch.device(device)
        self._lib = hostlib.lib()
        self._layouts: Dict[tuple, Dict[str, int]] = {}
        self._info = np.zeros(8, dtype=np.int32)
        self._pad_np = hostlib.i32([0])
        self.G = len(cache.paged)
        self.max_tokens, self.max_seqs, self.max_width = int(max_tokens), int(max_seqs), int(max_table_width)
        self.capacity = self._layout(self.max_tokens, self.max_seqs, self.max_width, self.max_tokens)["_total"]
        self.dev = torch.zeros(self.capacity, dtype=torch.int32, device=self.device)
        self.cuda = self.device.type == "cuda"
        self._ring = []
        for _ in range(ring if self.cuda else 1):
            host = torch.zeros(self.capacity, dtype=torch.int32, pin_memory=self.cuda)
            self._ring.append([host, torch.cuda.Event() if self.cuda else None, False])
        self._next = 0
        self.h2d_bytes_last = 0

    _NAMES = ("cu_q", "seqlens_k", "state_slots")

    def _layout(self, n_cap: int, s_cap: int, width: int, r_cap: int) -> Dict[str, int]:
        """Offsets of a step's arrays in the buffer (computed by the host runtime, which also
        fills them)."""
        key = (n_cap, s_cap, width, r_cap)
        lay = self._layouts.get(key)
        if lay is None:
            G = self.G
            raw = np.zeros(self._lib.vh_layout_len(G), dtype=np.int32)
            self._lib.vh_layout(G, n_cap, s_cap, width, r_cap, raw.ctypes.data)
            names = (["cu_q", "seqlens_k", "state_slots"] + [f"table{g}" for g in range(G)]
                     + ["tokens", "positions", "tok_seq"] + [f"slots{g}" for g in range(G)]
                     + ["rows", "token_src", "_total"])
            lay = dict(zip(names, raw.tolist()))
            if len(self._layouts) > 256:
                self._layouts.clear()
            self._layouts[key] = lay
        return lay

    def pack(self, entries: Sequence[StepEntry], dtype: torch.dtype, *, n_cap: Optional[int] = None,
             s_cap: Optional[int] = None, width: Optional[int] = None,
             status: Optional[torch.Tensor] = None, plan=None) -> StepContext:
        """Build the device context.  With capacities given, the step is padded to them:
        padding sequences hold one token at position 0 that writes to page 0's slot of a
        page the caller set aside (``pad_page``) and to the scratch state slot.  ``plan`` is a
        step the host runtime's scheduler has planned (its handle): the arrays are then taken
        from there and ``entries`` is not looked at."""
        cache = self.cache
        pad = n_cap is not None
        if plan is not None:
            S, n, R, w_need = plan.num_entries, plan.num_tokens, plan.num_rows, plan.width_needed
        else:
            S = len(entries)
            qlens = [len(e.tokens) for e in entries]
            n = sum(qlens)
            R = sum(len(e.want) for e in entries)
            w_need = max([cache.pages_for(e.start + q) for e, q in zip(entries, qlens)] or [1])
        n_c = n_cap if pad else n
        s_c = s_cap if pad else S
        w_c = width if width is not None else _round_up(w_need, 4)
        if n > n_c or S > s_c or w_need > w_c or n_c > self.max_tokens or s_c > self.max_seqs or w_c > self.max_width:
            raise StepError(f"step of {n} tokens / {S} sequences / {w_need} pages exceeds the packer's capacity "
                            f"({self.max_tokens} / {self.max_seqs} / {self.max_width})")
        r_c = n_c if pad else max(R, 1)
        lay = self._layout(n_c, s_c, w_c, r_c)
        total = lay["_total"]

        slot = self._ring[self._next]
        self._next = (self._next + 1) % len(self._ring)
        host, event, used = slot
        if used and event is not None:
            event.synchronize()
        info = self._info
        pads = self._pad_np.ctypes.data if (pad and S < s_c) else 0
        if pad and S < s_c and self._pad_pages is None:
            raise StepError("padding a step needs a page set aside for it")
        if plan is not None:
            rc = self._lib.vs_pack_plan(plan.handle, n_c, s_c, w_c, r_c, 1 if pad else 0, pads, cache.scratch_slot,
                                        host.data_ptr(), info.ctypes.data)
        else:
            handles = hostlib.i32([e.cache.handle for e in entries] or [0])
            ql = hostlib.i32(qlens or [0])
            toks = hostlib.i32([t for e in entries for t in e.tokens] or [0])
            wc = hostlib.i32([len(e.want) for e in entries] or [0])
            wants = hostlib.i32([w for e in entries for w in e.want] or [0])
            rc = self._lib.vh_pack(cache.native, S, handles.ctypes.data, ql.ctypes.data, toks.ctypes.data,
                                   wc.ctypes.data, wants.ctypes.data, n_c, s_c, w_c, r_c, 1 if pad else 0, pads,
                                   cache.scratch_slot, host.data_ptr(), info.ctypes.data)
        if rc != 0:
            raise StepError(f"the step cannot be packed: {hostlib.last_error()}")
        _, _, num_rows, max_q, max_k, identity = info[:6].tolist()

        if self.cuda:
            self.dev[:total].copy_(host[:total], non_blocking=True)
            event.record(torch.cuda.current_stream())
            slot[2] = True
        else:
            self.dev[:total].copy_(host[:total])
        self.h2d_bytes_last = total * 4

        d = self.dev
        n_eff, s_eff = (n_c, s_c) if pad else (n, S)

        def view(name: str, count: int) -> torch.Tensor:
            return d[lay[name]:lay[name] + count]

        groups = [GroupMeta(view(f"slots{g}", n_eff),
                            d[lay[f"table{g}"]:lay[f"table{g}"] + s_eff * w_c].view(s_eff, w_c))
                  for g in range(self.G)]
        return StepContext(
            n=n_eff, num_seqs=s_eff, num_rows=num_rows, max_q=max_q, max_k=max_k,
            tokens=view("tokens", n_eff), positions=view("positions", n_eff), tok_seq=view("tok_seq", n_eff),
            cu_q=view("cu_q", s_eff + 1), seqlens_k=view("seqlens_k", s_eff),
            state_slots=view("state_slots", s_eff),
            logits_rows=view("rows", num_rows) if num_rows else None,
            groups=groups, dtype=dtype, status=status, rows_identity=bool(identity) and num_rows == n_eff,
            token_src=view("token_src", n_eff), unknown_tokens=bool(plan is not None and plan.has_unknown))

    # a page per group that padding rows may scribble on; set by whoever captures graphs
    _pad_pages: Optional[List[int]] = None

    def set_pad_pages(self, pages: List[int]) -> None:
        self._pad_pages = list(pages)
        self._pad_np = hostlib.i32(list(pages) or [0])

    def pad_page(self, g: int) -> int:
        if self._pad_pages is None:
            raise StepError("padding a step needs a page set aside for it")
        return self._pad_pages[g]

    def pad_slot(self, g: int) -> int:
        return self.pad_page(g) * self.cache.page_size
