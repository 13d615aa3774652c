"""Token selection for the rows of a step.

Rows that are greedy, or temperature-only, are decided on the device in one launch (argmax,
Gumbel-max); penalties are applied on the device before it.  Rows that truncate the
distribution (top-k, min-p, top-p) are sampled on the host from their row of logits, with
the reference's pipeline (crates/vapi-engine/src/sampler.rs:162-180, 302-376): scale by
1/T, keep what lies within 30 nats of the maximum, softmax, sort by probability then id,
top-k, min-p, top-p, weighted choice.  Every request has a random generator and a draw
counter of its own, so a seeded request does not depend on what else is in the batch.
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

    @staticmethod
    def device_only(p: SamplingParams) -> bool:
        """Whether a row with these parameters is decided by the device launch alone (greedy, or
        temperature without truncation) and needs nothing of the host but the result."""
        return (p.is_greedy or p.device_drawable) and not p.has_penalties and p.logprobs is None

    def launch(self, logits: torch.Tensor, rows: Sequence[Tuple[SamplingParams, SamplerState]],
               out: torch.Tensor) -> PendingSample:
        """For rows that are all :meth:`device_only`: decide them on the device into ``out`` and
        start the copy to the host without waiting for it."""
        R = len(rows)
        assert logits.shape[0] >= R and all(self.device_only(p) for p, _ in rows)
        dev = logits.device
        self.h2d_bytes_last = 0
        if all(p.is_greedy for p, _ in rows):
            ops.sample_rows(logits[:R], out=out[:R])
        else:
            m64 = torch.empty((2, R), dtype=torch.int64)
            for r, (p, st) in enumerate(rows):
                m64[0, r] = st.seed - (1 << 64) if st.seed >= (1 << 63) else st.seed
                m64[1, r] = st.device_draws
                if not p.is_greedy:
                    st.device_draws += 1
            mode = torch.tensor([1 if p.is_greedy else 2 for p, _ in rows], dtype=torch.int32).to(dev)
            inv_t = torch.tensor([p.inv_temperature for p, _ in rows], dtype=torch.float32).to(dev)
            m64d = m64.to(dev)
            ops.sample_rows(logits[:R], mode, inv_t, m64d[0], m64d[1], out=out[:R])
            self.h2d_bytes_last += R * 24
        if not self._ring:
            for _ in range(3):
                self._ring.append([torch.zeros(max(self.max_rows, out.numel()), dtype=torch.int32, pin_memory=True),
                                   torch.cuda.Event()])
        host, event = self._ring[self._next]
        self._next = (self._next + 1) % len(self._ring)
        host[:R].copy_(out[:R], non_blocking=True)
        event.record(torch.cuda.current_stream())
        self.d2h_bytes_last = 4 * R
        return PendingSample(R, host, event)

    def finish(self, pending: PendingSample) -> List[int]:
        """Wait for a launched sample and return its tokens."""
        if pending.tokens is not None:
            return pending.tokens
        pending.event.synchronize()
        pending.tokens = pending.host[:pending.rows].tolist()
        return pending.tokens

    def sample(self, logits: torch.Tensor, rows: Sequence[Tuple[SamplingParams, SamplerState]]) -> List[int]:
        R = len(rows)
        assert logits.shape[0] >= R
        self.h2d_bytes_last = 0
        dev = logits.device
        # rows that report log-probabilities: their raw logits, before any penalty touches them
        raw: Dict[int, Tuple[float, List[Tuple[int, float]], np.ndarray]] = {}
        for r, (p, _) in enumerate(rows):
            if p.logprobs is not None:
                row = logits[r].to(torch.float32).cpu().numpy()
                lse, top = row_logprobs(row, p.logprobs)
                raw[r] = (lse, top, row)
        toks = self._choose(logits, rows, dev)
        self.last_logprobs = [TokenLogprobs(toks[r], float(raw[r][2][toks[r]]) - raw[r][0], raw[r][1]) if r in raw else None
                              for r in range(R)]
        return toks

    def _choose(self, logits: torch.Tensor, rows: Sequence[Tuple[SamplingParams, SamplerState]], dev) -> List[int]:
        R = len(rows)
        # penalties, on the device, for the rows that have any
        pr, pt, pc = [], [], []
        for r, (p, st) in enumerate(rows):
            if p.has_penalties and st.counts:
                for tok, cnt in st.counts.items():
                    pr.append(r); pt.append(tok); pc.append(float(cnt))
        if pr:
            rep = torch.tensor([p.repetition_penalty for p, _ in rows], dtype=torch.float32)
            frq = torch.tensor([p.frequency_penalty for p, _ in rows], dtype=torch.float32)
            prs = torch.tensor([p.presence_penalty for p, _ in rows], dtype=torch.float32)
            ops.apply_penalties(logits, torch.tensor(pr, dtype=torch.int32).to(dev), torch.tensor(pt, dtype=torch.int32).to(dev),
                                torch.tensor(pc, dtype=torch.float32).to(dev), rep.to(dev), frq.to(dev), prs.to(dev))
            self.h2d_bytes_last += 12 * len(pr) + 12 * R
        all_greedy = all(p.is_greedy for p, _ in rows)
        if all_greedy:
            out = ops.sample_rows(logits[:R])
            toks = out.cpu().tolist()
            self.d2h_bytes_last = 4 * R
            return [int(t) for t in toks]
        mode = [1 if p.is_greedy else (2 if p.device_drawable else 0) for p, _ in rows]
        inv_t = [p.inv_temperature for p, _ in rows]
        seeds = [st.seed - (1 << 64) if st.seed >= (1 << 63) else st.seed for _, st in rows]
        draws = [st.device_draws for _, st in rows]
        out = ops.sample_rows(logits[:R], torch.tensor(mode, dtype=torch.int32).to(dev),
                              torch.tensor(inv_t, dtype=torch.float32).to(dev),
                              torch.tensor(seeds, dtype=torch.int64).to(dev),
                              torch.tensor(draws, dtype=torch.int64).to(dev),
                              torch.zeros(R, dtype=torch.int32, device=dev))
        self.h2d_bytes_last += R * 24
        toks = [int(t) for t in out.cpu().tolist()]
        self.d2h_bytes_last = 4 * R
        for r, (p, st) in enumerate(rows):
            if mode[r] == 2:
                st.device_draws += 1
            elif mode[r] == 0:
                row = logits[r].to(torch.float32).cpu().numpy()
                self.d2h_bytes_last += row.nbytes
                toks[r] = host_sample(row, p, st)
        return toks
