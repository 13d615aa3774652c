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
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

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
    slot_mapping: torch.Tensor      # [n] int32: page * page_size + offset of each token
    block_table: torch.Tensor       # [S, width] int32


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

    def _layout(self, n_cap: int, s_cap: int, width: int, r_cap: int) -> Dict[str, int]:
        off, lay = 0, {}

        def put(name: str, count: int) -> None:
            nonlocal off
            lay[name] = off
            off += _round_up(max(count, 1), 4)

        put("cu_q", s_cap + 1)
        put("seqlens_k", s_cap)
        put("state_slots", s_cap)
        for g in range(self.G):
            put(f"table{g}", s_cap * width)
        put("tokens", n_cap)
        put("positions", n_cap)
        put("tok_seq", n_cap)
        for g in range(self.G):
            put(f"slots{g}", n_cap)
        put("rows", r_cap)
        lay["_total"] = off
        return lay

    def pack(self, entries: Sequence[StepEntry], dtype: torch.dtype, *, n_cap: Optional[int] = None,
             s_cap: Optional[int] = None, width: Optional[int] = None,
             status: Optional[torch.Tensor] = None) -> StepContext:
        """Build the device context.  With capacities given, the step is padded to them:
        padding sequences hold one token at position 0 that writes to page 0's slot of a
        page the caller set aside (``pad_page``) and to the scratch state slot."""
        cache, P = self.cache, self.cache.page_size
        S = len(entries)
        n = sum(len(e.tokens) for e in entries)
        R = sum(len(e.want) for e in entries)
        w_need = max([cache.pages_for(e.start + len(e.tokens)) for e in entries] or [1])
        pad = n_cap is not None
        n_c = n_cap if pad else n
        s_c = s_cap if pad else S
        w_c = width if width is not None else _round_up(w_need, 4)
        if n > n_c or S > s_c or w_need > w_c or n_c > self.max_tokens or s_c > self.max_seqs or w_c > self.max_width:
            raise StepError(f"step of {n} tokens / {S} sequences / {w_need} pages exceeds the packer's capacity "
                            f"({self.max_tokens} / {self.max_seqs} / {self.max_width})")
        lay = self._layout(n_c, s_c, w_c, n_c if pad else max(R, 1))
        total = lay["_total"]

        slot = self._ring[self._next]
        self._next = (self._next + 1) % len(self._ring)
        host, event, used = slot
        if used and event is not None:
            event.synchronize()
        hb = host.numpy()
        hb[:total] = 0

        cu_q, pos_n = [0], 0
        toks, poss, tseq, rows = [], [], [], []
        slots: List[List[int]] = [[] for _ in range(self.G)]
        max_q = max_k = 1 if pad else 0
        for si, e in enumerate(entries):
            q, st = len(e.tokens), e.start
            max_q, max_k = max(max_q, q), max(max_k, st + q)
            toks.extend(int(t) for t in e.tokens)
            poss.extend(range(st, st + q))
            tseq.extend([si] * q)
            rows.extend(pos_n + int(w) for w in e.want)
            for g in range(self.G):
                tb = e.cache.tables[g]
                if q == 1:
                    slots[g].append(tb[st // P] * P + st % P)
                else:
                    slots[g].extend(tb[p // P] * P + p % P for p in range(st, st + q))
                row = e.cache.table_row(g, w_c)
                o = lay[f"table{g}"] + si * w_c
                hb[o:o + row.size] = row
            hb[lay["seqlens_k"] + si] = st + q
            hb[lay["state_slots"] + si] = e.cache.slot
            pos_n += q
            cu_q.append(pos_n)
        # padding sequences of a fixed-shape step: one token each, nothing of theirs is read back
        for si in range(S, s_c):
            cu_q.append(cu_q[-1] + 1)
            hb[lay["seqlens_k"] + si] = 1
            hb[lay["state_slots"] + si] = cache.scratch_slot
            rows.append(len(toks))
            tseq.append(si)
            toks.append(0)
            poss.append(0)
            for g in range(self.G):
                slots[g].append(self.pad_slot(g))
                hb[lay[f"table{g}"] + si * w_c] = self.pad_page(g)
        n_tot = len(toks)
        hb[lay["cu_q"]:lay["cu_q"] + len(cu_q)] = cu_q
        hb[lay["tokens"]:lay["tokens"] + n_tot] = toks
        hb[lay["positions"]:lay["positions"] + n_tot] = poss
        hb[lay["tok_seq"]:lay["tok_seq"] + n_tot] = tseq
        for g in range(self.G):
            hb[lay[f"slots{g}"]:lay[f"slots{g}"] + n_tot] = slots[g]
        hb[lay["rows"]:lay["rows"] + len(rows)] = rows

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
            n=n_eff, num_seqs=s_eff, num_rows=len(rows), max_q=max_q, max_k=max_k,
            tokens=view("tokens", n_eff), positions=view("positions", n_eff), tok_seq=view("tok_seq", n_eff),
            cu_q=view("cu_q", s_eff + 1), seqlens_k=view("seqlens_k", s_eff),
            state_slots=view("state_slots", s_eff),
            logits_rows=view("rows", len(rows)) if rows else None,
            groups=groups, dtype=dtype, status=status, rows_identity=rows == list(range(n_eff)))

    # a page per group that padding rows may scribble on; set by whoever captures graphs
    _pad_pages: Optional[List[int]] = None

    def set_pad_pages(self, pages: List[int]) -> None:
        self._pad_pages = list(pages)

    def pad_page(self, g: int) -> int:
        if self._pad_pages is None:
            raise StepError("padding a step needs a page set aside for it")
        return self._pad_pages[g]

    def pad_slot(self, g: int) -> int:
        return self.pad_page(g) * self.cache.page_size
