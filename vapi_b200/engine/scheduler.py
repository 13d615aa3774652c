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

This is pure host logic: it touches the cache manager's bookkeeping and never a tensor.  The
decisions are made by the host runtime in C++ (``csrc/host.cpp``), which owns the sequences'
tokens and progress, the queues and the plan of the current step; the classes here are its
Python face and hold what C++ has no use for (request ids, sampling parameters).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Dict, List, Optional
from typing import Sequence as Seq

import numpy as np

from .. import hostlib
from ..cache.manager import CacheManager, RequestCache
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


_REASONS = {0: FinishReason.STOP, 1: FinishReason.LENGTH, 2: FinishReason.CANCELLED, 3: FinishReason.ERROR}
_REASON_CODES = {v: k for k, v in _REASONS.items()}
# fields of vs_seq_get
_STATUS, _PROMPT_LEN, _COMPUTED, _TARGET, _HANDLE, _PREEMPTIONS, _REASON, _TOTAL = range(8)
# lists of vs_list
(_L_SEQS, _L_HANDLES, _L_STARTS, _L_QLENS, _L_WANT_COUNTS, _L_WANTS, _L_TOKENS, _L_SAMPLED, _L_PREEMPTED,
 _L_STARTED, _L_RUNNING, _L_WAITING, _L_FINISHED) = range(13)


class Sequence:
    """One request's tokens and progress (crates/vapi-engine/src/sequence.rs), read through to
    the host runtime while the request lives and kept as a snapshot once it has been drained."""

    def __init__(self, sched: "Scheduler", seq_id: int, request_id, params: SamplingParams):
        self._sched, self.seq_id, self.request_id, self.params = sched, seq_id, request_id, params
        self.cache: Optional[RequestCache] = None
        self._snapshot: Optional[Dict[str, object]] = None

    def _get(self, field: int) -> int:
        return self._sched._lib.vs_seq_get(self._sched._h, self.seq_id, field)

    def _freeze(self) -> None:
        self._snapshot = {"tokens": self.tokens, "prompt_len": self.prompt_len, "num_computed": self.num_computed,
                          "prefill_target": self.prefill_target, "status": self.status,
                          "finish_reason": self.finish_reason, "preemptions": self.preemptions}

    def _field(self, name: str, field: int) -> int:
        if self._snapshot is not None:
            return self._snapshot[name]
        return self._get(field)

    @property
    def tokens(self) -> List[int]:
        if self._snapshot is not None:
            return self._snapshot["tokens"]
        return self._sched._seq_tokens(self.seq_id, 0)

    @property
    def prompt_len(self) -> int:
        return self._field("prompt_len", _PROMPT_LEN)

    @property
    def num_computed(self) -> int:
        return self._field("num_computed", _COMPUTED)

    @property
    def prefill_target(self) -> int:
        return self._field("prefill_target", _TARGET)

    @property
    def preemptions(self) -> int:
        return self._field("preemptions", _PREEMPTIONS)

    @property
    def status(self) -> SeqStatus:
        if self._snapshot is not None:
            return self._snapshot["status"]
        return SeqStatus(self._get(_STATUS))

    @property
    def finish_reason(self) -> Optional[FinishReason]:
        if self._snapshot is not None:
            return self._snapshot["finish_reason"]
        return _REASONS.get(self._get(_REASON))

    @property
    def total_len(self) -> int:
        if self._snapshot is not None:
            return len(self._snapshot["tokens"])
        return self._get(_TOTAL)

    @property
    def num_generated(self) -> int:
        return self.total_len - self.prompt_len

    @property
    def generated(self) -> List[int]:
        if self._snapshot is not None:
            return self._snapshot["tokens"][self.prompt_len:]
        return self._sched._seq_tokens(self.seq_id, self.prompt_len)

    def needs_prefill(self) -> bool:
        return self.num_computed < self.prefill_target

    def remaining_prefill(self) -> int:
        return max(0, self.prefill_target - self.num_computed)


class StepPlan:
    """The step the scheduler has planned.  The arrays live in the host runtime, which packs
    them for the device itself; ``entries`` builds the Python view of them on demand."""

    def __init__(self, sched: Optional["Scheduler"] = None, info: Seq[int] = (0,) * 9):
        self._sched = sched
        (self.num_entries, self.num_tokens, self.num_rows, n_pre, n_start, pure, self.width_needed, _,
         unknown) = info
        self.pure_decode = bool(pure)
        #: some token of this step is what the step before it samples and is not known yet
        self.has_unknown = bool(unknown)
        self.handle = sched._h if sched is not None else None
        self.batch_seqs: List[int] = sched._list(_L_SEQS, self.num_entries) if self.num_entries else []
        self.sampled_seqs: List[int] = sched._list(_L_SAMPLED, self.num_rows) if self.num_rows else []
        self.preempted: List[int] = sched._list(_L_PREEMPTED, n_pre) if n_pre else []
        self.started: List[int] = sched._list(_L_STARTED, n_start) if n_start else []
        self._entries: Optional[List[StepEntry]] = None
        self._caches: Optional[List[Optional[RequestCache]]] = None
        self._serial = sched._serial if sched is not None else 0

    def is_empty(self) -> bool:
        return self.num_entries == 0

    def _bind(self) -> None:
        """Remember which cache each entry belongs to (the faces can change at the next plan)."""
        self._caches = [self._sched.seqs[sid].cache for sid in self.batch_seqs]

    @property
    def entries(self) -> List[StepEntry]:
        if self._entries is None:
            if self._sched is not None and self._sched._serial != self._serial:
                raise RuntimeError("this plan's entries were not read before the next step was planned")
            out: List[StepEntry] = []
            if self.num_entries:
                s = self._sched
                qlens = s._list(_L_QLENS, self.num_entries)
                wants = s._list(_L_WANT_COUNTS, self.num_entries)
                tokens = s._list(_L_TOKENS, self.num_tokens)
                o = 0
                for rc, q, w in zip(self._caches, qlens, wants):
                    out.append(StepEntry(rc, tokens[o:o + q], [q - 1] if w else []))
                    o += q
            self._entries = out
        return self._entries

    def commit_cache(self) -> None:
        """What the step function does after it ran this step: every request of the step has
        computed its tokens."""
        if self.num_entries and self._sched._lib.vs_commit_cache(self.handle) != 0:
            raise RuntimeError(hostlib.last_error())


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, cache: CacheManager, eos_token_ids: Seq[int] = ()):
        self.cfg, self.cache = cfg, cache
        self.eos = tuple(int(e) for e in eos_token_ids)
        self.seqs: Dict[int, Sequence] = {}
        self._lib = hostlib.lib()
        eos = hostlib.i32(list(self.eos) or [0])
        self._h = self._lib.vs_new(cache.native, int(cfg.max_concurrent_seqs), int(cfg.max_batched_tokens),
                                   int(cfg.prefill_chunk_tokens), int(cfg.max_context), eos.ctypes.data, len(self.eos))
        self._info = np.zeros(9, dtype=np.int32)
        self._buf = np.zeros(1024, dtype=np.int32)
        self._seen_finished = 0
        self._serial = 0
        #: False: a plan's ``entries`` are built when it is planned; True (the engine loop):
        #: only if someone asks before the next plan, since the host runtime packs the step itself
        self.lazy_entries = False

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.vs_delete(h)

    # ---- reading the host runtime's lists ------------------------------------------------
    def _room(self, n: int) -> np.ndarray:
        if n > self._buf.size:
            self._buf = np.zeros(max(n, 2 * self._buf.size), dtype=np.int32)
        return self._buf

    def _list(self, which: int, count: int) -> List[int]:
        buf = self._room(count)
        n = self._lib.vs_list(self._h, which, buf.ctypes.data, buf.size)
        return buf[:n].tolist()

    def _seq_tokens(self, sid: int, start: int) -> List[int]:
        n = self._lib.vs_seq_get(self._h, sid, _TOTAL)
        buf = self._room(max(n, 1))
        k = self._lib.vs_seq_tokens(self._h, sid, start, buf.ctypes.data, buf.size)
        return buf[:max(k, 0)].tolist()

    @property
    def running(self) -> List[int]:
        return self._list(_L_RUNNING, self._lib.vs_counts(self._h, 0))

    @property
    def waiting(self) -> List[int]:
        return self._list(_L_WAITING, self._lib.vs_counts(self._h, 1))

    @property
    def finished(self) -> List[int]:
        return self._list(_L_FINISHED, self._lib.vs_counts(self._h, 2))

    # ---- admission ----------------------------------------------------------------------
    def admit(self, request_id, prompt: Seq[int], params: SamplingParams) -> int:
        params.validate()
        toks = hostlib.i32([int(t) for t in prompt] or [0])
        stop = hostlib.i32([int(t) for t in params.stop_token_ids] or [0])
        sid = self._lib.vs_admit(self._h, toks.ctypes.data, len(prompt), int(params.max_tokens),
                                 1 if params.ignore_eos else 0, stop.ctypes.data, len(params.stop_token_ids))
        if sid < 0:
            raise AdmitError(hostlib.last_error())
        self.seqs[sid] = Sequence(self, sid, request_id, params)
        return sid

    def admission_headroom(self) -> int:
        return max(0, self.cfg.max_concurrent_seqs - self.num_running - self.num_waiting)

    @property
    def num_waiting(self) -> int:
        return self._lib.vs_counts(self._h, 1)

    @property
    def num_running(self) -> int:
        return self._lib.vs_counts(self._h, 0)

    def is_idle(self) -> bool:
        return self.num_waiting == 0 and self.num_running == 0

    # ---- one step ---------------------------------------------------------------------
    def schedule(self) -> StepPlan:
        self._serial += 1
        self._lib.vs_schedule(self._h)
        self._lib.vs_plan_info(self._h, self._info.ctypes.data)
        info = self._info.tolist()
        plan = StepPlan(self, info)
        for sid in plan.preempted:
            self._drop_face(sid)
        for sid in plan.started:
            seq = self.seqs[sid]
            seq.cache = self.cache.adopt(sid, self._lib.vs_seq_get(self._h, sid, _HANDLE))
        if info[7] != self._seen_finished:
            self._note_finished()
        plan._bind()
        if not self.lazy_entries:
            plan.entries
        return plan

    def _drop_face(self, sid: int) -> None:
        seq = self.seqs.get(sid)
        if seq is not None and seq.cache is not None:
            self.cache.forget(seq.cache)
            seq.cache = None

    def _note_finished(self) -> None:
        """Requests the host runtime has retired since the last look no longer hold a cache."""
        ids = self.finished
        for sid in ids:
            self._drop_face(sid)
        self._seen_finished = len(ids)

    def commit(self, plan: StepPlan, sampled: Seq[int]) -> None:
        assert len(sampled) == len(plan.sampled_seqs)
        arr = hostlib.i32([int(t) for t in sampled] or [0])
        if self._lib.vs_commit(self._h, arr.ctypes.data, len(sampled)) != 0:
            raise RuntimeError(hostlib.last_error())
        if self._lib.vs_counts(self._h, 2) != self._seen_finished:
            self._note_finished()

    # ---- one step ahead ----------------------------------------------------------------
    def advance(self, plan: StepPlan) -> None:
        """The part of ``commit`` that does not depend on what was sampled: the requests of the
        planned step have computed their tokens, and each that asked for logits gains a token
        whose value is still unknown.  The next step can be planned after this."""
        if self._lib.vs_advance(self._h) != 0:
            raise RuntimeError(hostlib.last_error())

    def resolve(self, plan: StepPlan, sampled: Seq[int]) -> List[bool]:
        """The values of the tokens an advanced step produced, in the order of its
        ``sampled_seqs``; retires what finished.  Returns, per token, whether its request took
        it (a request that ended at an earlier token does not)."""
        assert len(sampled) == len(plan.sampled_seqs)
        took: List[bool] = []
        if sampled:
            ids = hostlib.i32(plan.sampled_seqs)
            arr = hostlib.i32([int(t) for t in sampled])
            acc = np.zeros(len(sampled), dtype=np.int32)
            self._lib.vs_resolve(self._h, ids.ctypes.data, arr.ctypes.data, len(sampled), acc.ctypes.data)
            took = acc.astype(bool).tolist()
        if self._lib.vs_counts(self._h, 2) != self._seen_finished:
            self._note_finished()
        return took

    def can_run_ahead(self) -> bool:
        """Whether the next step can be planned before the last one's tokens are known: no
        running request can run out of pages in it (a preemption would have to recompute
        tokens that are not known yet)."""
        return bool(self._lib.vs_can_run_ahead(self._h))

    def finish(self, sid: int, reason: FinishReason) -> None:
        self._lib.vs_finish(self._h, int(sid), _REASON_CODES[reason])
        self._note_finished()

    def cancel(self, sid: int) -> None:
        self.finish(sid, FinishReason.CANCELLED)

    def fail_all(self) -> List[int]:
        """A failed step fails every request in flight and frees what they hold; the
        scheduler goes on serving (crates/vapi-worker/src/engine.rs:622-650)."""
        buf = self._room(len(self.seqs) + 1)
        n = self._lib.vs_fail_all(self._h, buf.ctypes.data, buf.size)
        ids = buf[:n].tolist()
        self._note_finished()
        return ids

    def drain_finished(self) -> List[Sequence]:
        if self._lib.vs_counts(self._h, 2) == 0:
            return []
        out = []
        for sid in self.finished:
            seq = self.seqs.pop(sid, None)
            if seq is None:
                continue
            self._drop_face(sid)
            seq._freeze()
            self._lib.vs_erase(self._h, sid)
            out.append(seq)
        self._lib.vs_clear_finished(self._h)
        self._seen_finished = 0
        return out
