"""Token selection for the rows of a step.

Every row is decided on the device: greedy rows by argmax, temperature rows by the Gumbel-max
trick, and rows that cut the distribution (top-k, min-p, top-p) by the Gumbel-max trick over the
survivors of the cuts, which are the reference's (crates/vapi-engine/src/sampler.rs:162-180,
302-376: scale by 1/T, keep what lies within 30 nats of the maximum, top-k, min-p, top-p).
Penalties are applied on the device before that.  Which kernel decides a row depends on the
request's own parameters only, and the noise is keyed by the request's (seed, draw), so a seeded
request does not depend on what else is in the batch.  ``host_sample`` restates the reference's
host sampler (sort, cumulative sums, weighted choice with a generator per request); it is what
the device cuts are checked against and serves logits that live on the host.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from .params import SamplingParams

CANDIDATE_CUTOFF = 30.0


class SamplerState:
    """Per-request sampling state: occurrence counts for the penalties, the host generator,
    and the (seed, draw) pair that keys device-side noise."""

    def __init__(self, seed: Optional[int] = None):
        if seed is None:
            seed = int.from_bytes(os.urandom(8), "little")
        self.seed = int(seed) & 0xFFFF_FFFF_FFFF_FFFF
        self.rng = np.random.Generator(np.random.Philox(self.seed))
        self.counts: Dict[int, int] = {}
        self.device_draws = 0

    def observe(self, token: int) -> None:
        self.counts[token] = self.counts.get(token, 0) + 1

    def observe_all(self, tokens: Sequence[int]) -> None:
        for t in tokens:
            self.observe(int(t))


def penalise(l: float, count: int, p: SamplingParams) -> float:
    """Repetition is multiplicative and sign-aware, frequency scales with the count,
    presence applies once (crates/vapi-engine/src/sampler.rs:249-260)."""
    if p.repetition_penalty != 1.0:
        l = l / p.repetition_penalty if l > 0.0 else l * p.repetition_penalty
    l -= p.frequency_penalty * count
    if count > 0:
        l -= p.presence_penalty
    return l


def host_sample(logits: np.ndarray, p: SamplingParams, state: SamplerState) -> int:
    """One token from a float32 row on the host (penalties already applied)."""
    if p.is_greedy:
        return int(np.argmax(logits))            # the first index wins ties
    inv_t = np.float32(1.0 / max(p.temperature, 1e-5))
    scaled = logits.astype(np.float32) * inv_t
    mx = scaled.max()
    keep = np.nonzero(scaled >= mx - np.float32(CANDIDATE_CUTOFF))[0]
    e = np.exp(scaled[keep] - mx).astype(np.float32)
    s = e.sum(dtype=np.float32)
    prob = e / s if s > 0 else e
    order = np.lexsort((keep, -prob))            # probability descending, then id ascending
    ids, prob = keep[order], prob[order]
    if p.top_k is not None:
        k = max(int(p.top_k), 1)
        ids, prob = ids[:k], prob[:k]
    if p.min_p > 0.0 and len(prob):
        floor = np.float32(p.min_p) * prob[0]
        n = max(int(np.sum(np.cumprod(prob >= floor))), 1)
        ids, prob = ids[:n], prob[:n]
    if p.top_p < 1.0:
        cum = np.cumsum(prob, dtype=np.float32)
        n = int(np.searchsorted(cum, np.float32(p.top_p), side="left")) + 1
        n = max(min(n, len(prob)), 1)
        ids, prob = ids[:n], prob[:n]
    total = float(prob.sum(dtype=np.float32))
    if total <= 0.0:
        return int(ids[0]) if len(ids) else 0
    r = float(state.rng.random(dtype=np.float32)) * total
    acc = np.cumsum(prob, dtype=np.float32)
    i = int(np.searchsorted(acc, np.float32(r), side="left"))
    return int(ids[min(i, len(ids) - 1)])


@dataclass
class TokenLogprobs:
    """Log-probabilities at one generated position under the model's own distribution (the raw
    logits, before temperature and penalties: crates/vapi-engine/src/sampler.rs:114-153)."""
    token: int
    logprob: float
    top: List[Tuple[int, float]]        # the k most likely tokens, most likely first, ties by lower id


def row_logprobs(logits: np.ndarray, k: int):
    """``(lse, top)`` of a float32 row: log-sum-exp, and the k largest as (token, logprob)."""
    row = logits.astype(np.float32)
    mx = np.float32(row.max())
    lse = float(mx + np.log(np.exp(row - mx, dtype=np.float32).sum(dtype=np.float32)))
    top: List[Tuple[int, float]] = []
    if k > 0:
        k = min(k, row.size)
        cand = np.argpartition(-row, k - 1)[:k] if k < row.size else np.arange(row.size)
        # everything tied with the k-th value must compete, so that the lower id wins a tie
        cand = np.nonzero(row >= row[cand].min())[0]
        order = np.lexsort((cand, -row[cand]))[:k]
        top = [(int(cand[i]), float(row[cand[i]]) - lse) for i in order]
    return lse, top


@dataclass
class PendingSample:
    """Tokens decided on the device and on their way to the host."""
    rows: int
    host: Optional[torch.Tensor] = None         # pinned int32 buffer the copy lands in
    event: Optional["torch.cuda.Event"] = None
    tokens: Optional[List[int]] = None          # set when the tokens are already on the host
    with_status: bool = False                   # the copy starts with the kernels' status word
    status: int = 0                             # that word, once :meth:`Sampler.finish` has read it


class Sampler:
    """Decides the tokens of a step's rows.  Holds small persistent device buffers so that
    a step costs one upload, one launch (two with penalties) and one download."""

    def __init__(self, device, max_rows: int = 256):
        self.device = torch.device(device)
        self.max_rows = int(max_rows)
        self.d2h_bytes_last = 0
        self.h2d_bytes_last = 0
        self._ring: List[list] = []
        self._next = 0
        #: per row of the last :meth:`sample` call: None, or the :class:`TokenLogprobs` it asked for
        self.last_logprobs: List[Optional[TokenLogprobs]] = []
        #: the kernels' status word as the last :meth:`sample` call read it (0 without a status block)
        self.last_status = 0
        self._out: Optional[torch.Tensor] = None

    @staticmethod
    def device_only(p: SamplingParams) -> bool:
        """Whether the host has nothing to do for a row with these parameters but read the
        result: no penalties (their counts are uploaded each step) and no logprobs (the raw row
        is read back)."""
        return not p.has_penalties and p.logprobs is None

    def _ring_entry(self, out: torch.Tensor):
        """The next set of pinned staging buffers (results, per-row sampling data) with the event
        that says the copies of their last use are done."""
        if not self._ring:
            cap = max(self.max_rows, out.numel()) + 1
            for _ in range(3):
                self._ring.append([torch.zeros(cap, dtype=torch.int32, pin_memory=True),
                                   torch.zeros(cap * self._META_BYTES, dtype=torch.uint8, pin_memory=True),
                                   torch.cuda.Event(), False])
            self._meta_dev = torch.zeros(cap * self._META_BYTES, dtype=torch.uint8, device=out.device)
        entry = self._ring[self._next]
        self._next = (self._next + 1) % len(self._ring)
        if entry[3]:
            entry[2].synchronize()
        return entry

    #: bytes of sampling data per row: seed, draw (int64), 1/T, top_p, min_p (float32), mode, top_k (int32)
    _META_BYTES = 36

    def launch(self, logits: torch.Tensor, rows: Sequence[Tuple[SamplingParams, SamplerState]],
               out: torch.Tensor, status_block: Optional[torch.Tensor] = None) -> PendingSample:
        """Decide every row on the device into ``out`` (penalties, if any, must already have been
        applied to ``logits``) and start the copy to the host without waiting for it.

        ``status_block`` is a buffer whose first word is the kernels' status word and whose rest is
        ``out``: the word then comes to the host in the same copy as the tokens, so whoever reads
        the tokens learns at no cost whether a kernel of the step refused to go on."""
        R = len(rows)
        assert logits.shape[0] >= R
        if status_block is not None and (status_block.dtype != torch.int32
                                         or status_block.data_ptr() + 4 != out.data_ptr()):
            raise ValueError("the status block must be the int32 word right before the output tokens")
        entry = self._ring_entry(out)
        host, meta_host, event = entry[0], entry[1], entry[2]
        self.h2d_bytes_last = 0
        if all(p.is_greedy for p, _ in rows):
            ops.sample_rows(logits[:R], out=out[:R])
        else:
            # every row's sampling data in one pinned buffer and one upload: [seeds | draws | 1/T |
            # top_p | min_p | mode | top_k], each an array over the rows
            mb = meta_host.numpy()
            i64 = mb[:16 * R].view(np.int64).reshape(2, R)
            f32 = mb[16 * R:28 * R].view(np.float32).reshape(3, R)
            i32 = mb[28 * R:36 * R].view(np.int32).reshape(2, R)
            plain = cut = False
            for r, (p, st) in enumerate(rows):
                i64[0, r] = st.seed - (1 << 64) if st.seed >= (1 << 63) else st.seed
                i64[1, r] = st.device_draws
                f32[0, r], f32[1, r], f32[2, r] = p.inv_temperature, p.top_p, p.min_p
                if p.is_greedy:
                    i32[0, r], i32[1, r] = 1, -1
                    plain = True
                elif p.device_drawable:                   # nothing but temperature
                    i32[0, r], i32[1, r] = 2, -1
                    st.device_draws += 1
                    plain = True
                else:                                     # cut by top-k / min-p / top-p: the other kernel
                    i32[0, r], i32[1, r] = 0, (p.top_k or 0)
                    st.device_draws += 1
                    cut = True
            md = self._meta_dev
            md[:36 * R].copy_(meta_host[:36 * R], non_blocking=True)
            self.h2d_bytes_last += 36 * R
            d64 = md[:16 * R].view(torch.int64).view(2, R)
            d32f = md[16 * R:28 * R].view(torch.float32).view(3, R)
            d32i = md[28 * R:36 * R].view(torch.int32).view(2, R)
            if plain:
                ops.sample_rows(logits[:R], d32i[0], d32f[0], d64[0], d64[1], out=out[:R])
            if cut:
                ops.sample_truncated(logits[:R], d32f[0], d32i[1], d32f[1], d32f[2], d64[0], d64[1], out=out[:R])
        if status_block is not None:
            host[:R + 1].copy_(status_block[:R + 1], non_blocking=True)
        else:
            host[:R].copy_(out[:R], non_blocking=True)
        event.record(torch.cuda.current_stream())
        entry[3] = True
        self.d2h_bytes_last = 4 * (R + (status_block is not None))
        return PendingSample(R, host, event, with_status=status_block is not None)

    def finish(self, pending: PendingSample) -> List[int]:
        """Wait for a launched sample and return its tokens."""
        if pending.tokens is not None:
            return pending.tokens
        pending.event.synchronize()
        if pending.with_status:
            words = pending.host[:pending.rows + 1].tolist()
            pending.status, pending.tokens = words[0], words[1:]
        else:
            pending.tokens = pending.host[:pending.rows].tolist()
        return pending.tokens

    def sample(self, logits: torch.Tensor, rows: Sequence[Tuple[SamplingParams, SamplerState]],
               out: Optional[torch.Tensor] = None, status_block: Optional[torch.Tensor] = None) -> List[int]:
        """Tokens for the rows of a step, waiting for them: raw rows are read back for requests
        that report logprobs, penalties are applied on the device, and every row is then decided
        as :meth:`launch` decides it (logits on the host: by the host restatement).  ``out`` and
        ``status_block`` as for :meth:`launch`; the status word read is left in ``last_status``."""
        R = len(rows)
        assert logits.shape[0] >= R
        dev = logits.device
        # rows that report log-probabilities: their raw logits, before any penalty touches them
        raw: Dict[int, Tuple[float, List[Tuple[int, float]], np.ndarray]] = {}
        for r, (p, _) in enumerate(rows):
            if p.logprobs is not None:
                row = logits[r].to(torch.float32).cpu().numpy()
                lse, top = row_logprobs(row, p.logprobs)
                raw[r] = (lse, top, row)
        extra_h2d = self._penalise(logits, rows, dev)
        if logits.is_cuda:
            if out is None or out.numel() < R:
                if self._out is None or self._out.numel() < R or self._out.device != dev:
                    self._out = torch.zeros(max(self.max_rows, R), dtype=torch.int32, device=dev)
                out, status_block = self._out, None
            pending = self.launch(logits, rows, out, status_block)
            toks = self.finish(pending)
            self.last_status = pending.status
            self.h2d_bytes_last += extra_h2d
        else:
            toks = self._choose_on_host(logits, rows)
        self.last_logprobs = [TokenLogprobs(toks[r], float(raw[r][2][toks[r]]) - raw[r][0], raw[r][1]) if r in raw else None
                              for r in range(R)]
        return toks

    def _penalise(self, logits: torch.Tensor, rows, dev) -> int:
        """Penalties on the device for the rows that have any; returns the bytes uploaded."""
        pr, pt, pc = [], [], []
        for r, (p, st) in enumerate(rows):
            if p.has_penalties and st.counts:
                for tok, cnt in st.counts.items():
                    pr.append(r); pt.append(tok); pc.append(float(cnt))
        if not pr:
            return 0
        R = len(rows)
        rep = torch.tensor([p.repetition_penalty for p, _ in rows], dtype=torch.float32)
        frq = torch.tensor([p.frequency_penalty for p, _ in rows], dtype=torch.float32)
        prs = torch.tensor([p.presence_penalty for p, _ in rows], dtype=torch.float32)
        ops.apply_penalties(logits, torch.tensor(pr, dtype=torch.int32).to(dev), torch.tensor(pt, dtype=torch.int32).to(dev),
                            torch.tensor(pc, dtype=torch.float32).to(dev), rep.to(dev), frq.to(dev), prs.to(dev))
        return 12 * len(pr) + 12 * R

    def _choose_on_host(self, logits: torch.Tensor, rows) -> List[int]:
        """Logits that live on the host (tests of the host logic): greedy and plain temperature
        through the kernels' stand-ins, cuts through the host restatement of the sampler."""
        R = len(rows)
        mode = [1 if p.is_greedy else (2 if p.device_drawable else 0) for p, _ in rows]
        inv_t = [p.inv_temperature for p, _ in rows]
        seeds = [st.seed - (1 << 64) if st.seed >= (1 << 63) else st.seed for _, st in rows]
        draws = [st.device_draws for _, st in rows]
        out = ops.sample_rows(logits[:R], torch.tensor(mode, dtype=torch.int32), torch.tensor(inv_t, dtype=torch.float32),
                              torch.tensor(seeds, dtype=torch.int64), torch.tensor(draws, dtype=torch.int64),
                              torch.zeros(R, dtype=torch.int32))
        toks = [int(t) for t in out.tolist()]
        self.d2h_bytes_last = 4 * R
        for r, (p, st) in enumerate(rows):
            if mode[r] == 2:
                st.device_draws += 1
            elif mode[r] == 0:
                toks[r] = host_sample(logits[r].to(torch.float32).numpy(), p, st)
        return toks
