"""Continuous-batching scheduler: admission, prompt portions under a token budget,
decoding, finishing, and what happens when pages run out.

Behaviour follows the reference's scheduler (crates/vapi-engine/src/scheduler.rs,
sequence.rs) without its prefix cache and forks:

* ``admit`` queues a request; an empty prompt or one at or beyond ``max_context`` is refused;
* ``schedule`` builds one step: decode tokens of running requests first (one each), then
  the next portions of prompts already started, then waiting requests in FIFO order while
  budget, request slots and pages (watermark-checked) allow.  A request that cannot start
  goes back to the *front* of the queue and admission stops, so small requests cannot
  starve a large one;
* a portion is ``min(remaining prompt, prefill_chunk_tokens, budget)`` tokens; only the
  portion that completes the known text asks for logits;
* **when pages run out** for a running request (a decode token that crosses into a new
  page, or a portion), the request is *preempted by recompute*: everything it holds (pages
  and state slot) is given back, it keeps its generated tokens, and it returns to the front
  of the queue to be prefilled again, prompt plus generated text, in portions;
* ``commit`` advances every request of the step, appends sampled tokens and retires what
  finished: EOS (only after at least one generated token) or a stop token id -> STOP;
  ``max_tokens`` or the context limit -> LENGTH.

This is pure host logic: it touches the cache manager's bookkeeping and never a tensor.
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple
from typing import Sequence as Seq

from ..cache.manager import CacheManager, RequestCache
from ..cache.pool import OutOfSlots
from ..sampling.params import FinishReason, SamplingParams
from .step import StepEntry


class AdmitError(ValueError):
    pass


class SeqStatus(enum.Enum):
    WAITING = 0
    PREFILLING = 1
    DECODING = 2
    FINISHED = 3


@dataclass
class SchedulerConfig:
    """Names and defaults of the reference's ``[worker]`` / ``[cache]`` / ``[model]`` options
    (crates/vapi-engine/src/scheduler.rs:10-30, crates/vapi-core/src/config.rs:175-190, 259)."""
    max_concurrent_seqs: int = 64
    max_batched_tokens: int = 8192
    prefill_chunk_tokens: int = 2048
    max_context: int = 8192


class Sequence:
    """One request's tokens and progress (crates/vapi-engine/src/sequence.rs)."""

    def __init__(self, seq_id: int, request_id, prompt: Seq[int], params: SamplingParams):
        self.seq_id, self.request_id, self.params = seq_id, request_id, params
        self.tokens: List[int] = [int(t) for t in prompt]
        self.prompt_len = len(self.tokens)
        self.num_computed = 0
        self.prefill_target = self.prompt_len   # known text to push through in portions
        self.status = SeqStatus.WAITING
        self.finish_reason: Optional[FinishReason] = None
        self.cache: Optional[RequestCache] = None
        self.preemptions = 0

    @property
    def total_len(self) -> int:
        return len(self.tokens)

    @property
    def num_generated(self) -> int:
        return len(self.tokens) - self.prompt_len

    @property
    def generated(self) -> List[int]:
        return self.tokens[self.prompt_len:]

    def needs_prefill(self) -> bool:
        return self.num_computed < self.prefill_target

    def remaining_prefill(self) -> int:
        return max(0, self.prefill_target - self.num_computed)

    def reset_for_recompute(self) -> None:
        """After preemption: keep every token, compute again from position 0
        (sequence.rs:167-176)."""
        self.num_computed = 0
        self.prefill_target = len(self.tokens)
        self.status = SeqStatus.WAITING
        self.cache = None
        self.preemptions += 1

    def check_finished(self, eos: Seq[int], max_context: int) -> Optional[FinishReason]:
        """sequence.rs:179-202."""
        if self.num_generated > 0:
            last = self.tokens[-1]
            if (not self.params.ignore_eos and last in eos) or last in self.params.stop_token_ids:
                return FinishReason.STOP
        if self.num_generated >= self.params.max_tokens:
            return FinishReason.LENGTH
        if self.total_len >= max_context:
            return FinishReason.LENGTH
        return None


@dataclass
class StepPlan:
    entries: List[StepEntry] = field(default_factory=list)
    batch_seqs: List[int] = field(default_factory=list)        # sequence of each entry
    sampled_seqs: List[int] = field(default_factory=list)      # sequence behind each wanted row, in row order
    preempted: List[int] = field(default_factory=list)
    started: List[int] = field(default_factory=list)

    def is_empty(self) -> bool:
        return not self.entries

    @property
    def num_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, cache: CacheManager, eos_token_ids: Seq[int] = ()):
        self.cfg, self.cache = cfg, cache
        self.eos = tuple(int(e) for e in eos_token_ids)
        self.seqs: Dict[int, Sequence] = {}
        self.waiting: Deque[int] = deque()
        self.running: List[int] = []
        self.finished: List[int] = []
        self._next_id = 0

    # ---- admission ----------------------------------------------------------------------
    def admit(self, request_id, prompt: Seq[int], params: SamplingParams) -> int:
        params.validate()
        if len(prompt) == 0:
            raise AdmitError("the prompt is empty")
        if len(prompt) >= self.cfg.max_context:
            raise AdmitError(f"the prompt has {len(prompt)} tokens; the context limit is {self.cfg.max_context}")
        if self.cache.paged and self.cache.pages_for(len(prompt) + 1) > min(g.pool.num_pages for g in self.cache.paged):
            raise AdmitError(f"the prompt has {len(prompt)} tokens; the whole cache holds fewer")
        sid = self._next_id
        self._next_id += 1
        self.seqs[sid] = Sequence(sid, request_id, prompt, params)
        self.waiting.append(sid)
        return sid

    def admission_headroom(self) -> int:
        return max(0, self.cfg.max_concurrent_seqs - len(self.running) - len(self.waiting))

    @property
    def num_waiting(self) -> int:
        return len(self.waiting)

    @property
    def num_running(self) -> int:
        return len(self.running)

    def is_idle(self) -> bool:
        return not self.waiting and not self.running

    # ---- one step ---------------------------------------------------------------------
    def schedule(self) -> StepPlan:
        plan = StepPlan()
        budget = self.cfg.max_batched_tokens
        budget = self._schedule_decodes(plan, budget)
        self._schedule_prefills(plan, budget)
        return plan

    def _schedule_decodes(self, plan: StepPlan, budget: int) -> int:
        survivors = []
        for sid in list(self.running):
            seq = self.seqs.get(sid)
            if seq is None or seq.status == SeqStatus.FINISHED:
                continue
            if seq.needs_prefill() or budget == 0:
                survivors.append(sid)
                continue
            if self.cache.reserve(seq.cache, seq.num_computed + 1):
                self._push(seq, 1, plan)
                budget -= 1
                survivors.append(sid)
            else:
                self._preempt(seq)
                plan.preempted.append(sid)
        self.running = survivors
        return budget

    def _schedule_prefills(self, plan: StepPlan, budget: int) -> None:
        for sid in list(self.running):
            if budget == 0:
                return
            seq = self.seqs.get(sid)
            if seq is None or not seq.needs_prefill() or seq.status == SeqStatus.FINISHED:
                continue
            budget = self._prefill_chunk(seq, plan, budget)
        while budget > 0 and len(self.running) < self.cfg.max_concurrent_seqs and self.waiting:
            sid = self.waiting.popleft()
            seq = self.seqs.get(sid)
            if seq is None or seq.status == SeqStatus.FINISHED:
                continue
            if not self._can_ever_fit(seq):
                # grown (by generation, then preemption) beyond what the whole cache holds
                self.finish(sid, FinishReason.LENGTH)
                continue
            if not self._try_start(seq):
                self.waiting.appendleft(sid)
                return
            plan.started.append(sid)
            self.running.append(sid)
            budget = self._prefill_chunk(seq, plan, budget)

    def _can_ever_fit(self, seq: Sequence) -> bool:
        need = self.cache.pages_for(seq.prefill_target + 1)
        return all(need + g.pool.watermark <= g.pool.num_pages for g in self.cache.paged)

    def _try_start(self, seq: Sequence) -> bool:
        """Pages for the known text plus its first generated token, watermark-checked, and
        a state slot (scheduler.rs:435-491)."""
        if not self.cache.can_admit(seq.prefill_target + 1):
            return False
        try:
            rc = self.cache.open(seq.seq_id)
        except OutOfSlots:
            return False
        if not self.cache.reserve(rc, seq.prefill_target + 1, guarded=True):
            self.cache.close(rc)
            return False
        seq.cache = rc
        seq.status = SeqStatus.PREFILLING
        return True

    def _prefill_chunk(self, seq: Sequence, plan: StepPlan, budget: int) -> int:
        q = min(seq.remaining_prefill(), self.cfg.prefill_chunk_tokens, budget)
        if q == 0:
            return budget
        if not self.cache.reserve(seq.cache, seq.num_computed + q):
            self._preempt(seq)
            plan.preempted.append(seq.seq_id)
            return budget
        self._push(seq, q, plan)
        return budget - q

    def _push(self, seq: Sequence, q: int, plan: StepPlan) -> None:
        start = seq.num_computed
        assert seq.cache is not None and seq.cache.num_tokens == start
        completes = start + q >= seq.total_len
        plan.entries.append(StepEntry(seq.cache, seq.tokens[start:start + q], [q - 1] if completes else []))
        plan.batch_seqs.append(seq.seq_id)
        if completes:
            plan.sampled_seqs.append(seq.seq_id)

    def _preempt(self, seq: Sequence) -> None:
        if seq.cache is not None:
            self.cache.close(seq.cache)
        seq.reset_for_recompute()
        if seq.seq_id in self.running:
            self.running.remove(seq.seq_id)
        self.waiting.appendleft(seq.seq_id)

    def commit(self, plan: StepPlan, sampled: Seq[int]) -> None:
        assert len(sampled) == len(plan.sampled_seqs)
        for sid, e in zip(plan.batch_seqs, plan.entries):
            seq = self.seqs.get(sid)
            if seq is None or seq.status == SeqStatus.FINISHED:
                continue
            seq.num_computed += len(e.tokens)
            if not seq.needs_prefill() and seq.status == SeqStatus.PREFILLING:
                seq.status = SeqStatus.DECODING
        for sid, tok in zip(plan.sampled_seqs, sampled):
            seq = self.seqs.get(sid)
            if seq is None or seq.status == SeqStatus.FINISHED:
                continue
            seq.tokens.append(int(tok))
            seq.prefill_target = max(seq.prefill_target, seq.num_computed)
            reason = seq.check_finished(self.eos, self.cfg.max_context)
            if reason is not None:
                self.finish(sid, reason)

    def finish(self, sid: int, reason: FinishReason) -> None:
        seq = self.seqs.get(sid)
        if seq is None or seq.status == SeqStatus.FINISHED:
            return
        seq.status = SeqStatus.FINISHED
        seq.finish_reason = reason
        if seq.cache is not None:
            self.cache.close(seq.cache)
            seq.cache = None
        if sid in self.running:
            self.running.remove(sid)
        if sid in self.waiting:
            self.waiting.remove(sid)
        self.finished.append(sid)

    def cancel(self, sid: int) -> None:
        self.finish(sid, FinishReason.CANCELLED)

    def fail_all(self) -> List[int]:
        """A failed step fails every request in flight and frees what they hold; the
        scheduler goes on serving (crates/vapi-worker/src/engine.rs:622-650)."""
        ids = [s for s in list(self.running) + list(self.waiting)]
        for sid in ids:
            self.finish(sid, FinishReason.ERROR)
        return ids

    def drain_finished(self) -> List[Sequence]:
        out = [self.seqs.pop(sid) for sid in self.finished if sid in self.seqs]
        self.finished = []
        return out
