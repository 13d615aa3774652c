"""The engine loop: scheduler + step function + sampler.

One ``step()`` is what the reference's ``Engine::step`` does
(crates/vapi-worker/src/engine.rs:653-1088) without text handling: plan a batch, run it,
choose a token for every row that asked for logits, commit, report what finished.  A step
function that raises fails every request in flight, frees what they hold, and leaves the
engine able to serve the next request (engine.rs:622-650); after ``max_step_failures``
failures in a row the error is passed on (crates/vapi-worker/src/runner.rs:210-235).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..sampling.params import FinishReason, SamplingParams
from ..sampling.sampler import PendingSample, Sampler, SamplerState, TokenLogprobs
from .runner import ModelRunner
from .scheduler import AdmitError, Scheduler, SchedulerConfig, StepPlan


@dataclass
class Finished:
    request_id: object
    prompt_tokens: int
    tokens: List[int]
    reason: FinishReason
    preemptions: int = 0
    logprobs: Optional[List[TokenLogprobs]] = None     # one per generated token, when the request asked


@dataclass
class StepOutput:
    new_tokens: Dict[object, int] = field(default_factory=dict)   # request id -> token sampled this step
    finished: List[Finished] = field(default_factory=list)
    did_work: bool = False
    num_tokens: int = 0
    preempted: int = 0


@dataclass
class EngineStats:
    steps: int = 0
    tokens_in: int = 0
    tokens_out: int = 0
    preemptions: int = 0
    failed_steps: int = 0
    ahead_steps: int = 0          # steps that were enqueued before the step before them had been read
    schedule_ms: float = 0.0
    forward_ms: float = 0.0
    sample_ms: float = 0.0
    commit_ms: float = 0.0


class Engine:
    """``run_ahead`` (on by default on a CUDA device): while the host has nothing to do for any
    live request but read its token (no penalties, no logprobs), a step is enqueued
    before the tokens of the step before it have been read: its input tokens are fetched on the
    device from that step's sampled output, and the host reads results one step late, while
    the next step already runs.  ``step()`` then reports the tokens of the step before.  A
    request that ends on EOS or a stop id has taken part in one more step, whose result for it is
    dropped.  Every token is computed from the same inputs as without running ahead; only the
    batch of a step can be one row larger, which in bfloat16 may take another kernel and so
    another rounding (in float32 the tokens are identical)."""

    def __init__(self, runner: ModelRunner, cfg: Optional[SchedulerConfig] = None, *,
                 max_step_failures: int = 3, use_graphs: bool = True, run_ahead: Optional[bool] = None):
        self.runner = runner
        cfg = cfg or SchedulerConfig()
        cfg.max_context = min(cfg.max_context, runner.max_context)
        cfg.max_batched_tokens = min(cfg.max_batched_tokens, runner.max_batched_tokens)
        cfg.max_concurrent_seqs = min(cfg.max_concurrent_seqs, runner.cache.max_requests)
        self.cfg = cfg
        self.scheduler = Scheduler(cfg, runner.cache, runner.plan.eos_token_ids)
        self.scheduler.lazy_entries = True
        self.sampler = Sampler(runner.device)
        self.states: Dict[int, SamplerState] = {}
        self.stats = EngineStats()
        self.max_step_failures = int(max_step_failures)
        self._failures_in_a_row = 0
        self.last_error: Optional[str] = None
        self.use_graphs = use_graphs
        on_cuda = torch.device(runner.device).type == "cuda"
        self.run_ahead = on_cuda if run_ahead is None else (bool(run_ahead) and on_cuda)
        self._inflight: Optional[Tuple[StepPlan, PendingSample]] = None
        self._needs_host: set = set()          # live requests whose rows the host has to sample
        self._logprobs: Dict[int, List[TokenLogprobs]] = {}
        #: replaceable in tests: the function that runs a planned batch and returns logits
        self.step_fn: Callable[[StepPlan], Optional[torch.Tensor]] = self._run

    # ---- requests -------------------------------------------------------------------------
    def admit(self, request_id, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        for t in prompt:
            if not 0 <= int(t) < self.runner.vocab_size:
                raise AdmitError(f"token {t} is outside the vocabulary of {self.runner.vocab_size}")
        sid = self.scheduler.admit(request_id, prompt, params)
        st = SamplerState(params.seed)
        if params.has_penalties:
            st.observe_all(prompt)
        self.states[sid] = st
        if not Sampler.device_only(params):
            self._needs_host.add(sid)
        if params.logprobs is not None:
            self._logprobs[sid] = []
        return sid

    def cancel(self, sid: int) -> None:
        self.scheduler.cancel(sid)

    def is_idle(self) -> bool:
        return self.scheduler.is_idle() and not self.scheduler.finished and self._inflight is None

    # ---- one step ---------------------------------------------------------------------
    def _run(self, plan: StepPlan) -> Optional[torch.Tensor]:
        if self.use_graphs and plan.pure_decode and hasattr(self.runner, "step_decode_graph"):
            out = self.runner.step_decode_graph(None, plan=plan)
            if out is not None:
                return out
        return self.runner.step(None, plan=plan)

    def _can_run_ahead(self) -> bool:
        return self.run_ahead and not self._needs_host and self.scheduler.can_run_ahead()

    def _resolve(self, plan: StepPlan, pending: PendingSample, out: StepOutput) -> None:
        """Read a step's sampled tokens, hand them to the scheduler and report them.  The
        kernels' status word comes with the tokens: if a kernel of the step (or of any step
        since the word was last read) refused an index or gave up a wait, the tokens are not
        trusted and the step counts as failed."""
        toks = self.sampler.finish(pending)
        self._check_status(pending.status)
        took = self.scheduler.resolve(plan, toks)
        for sid, tok, ok in zip(plan.sampled_seqs, toks, took):
            if not ok:
                continue
            st = self.states.get(sid)
            if st is not None:
                st.observe(tok)
            seq = self.scheduler.seqs.get(sid)
            if seq is not None:
                out.new_tokens[seq.request_id] = tok
        self.stats.tokens_out += sum(took)

    def _check_status(self, code: int) -> None:
        """Raise for a non-zero status word.  On a CUDA device the word is the one that came to
        the host with the sampled tokens; a device whose memory the host can read is asked
        directly."""
        status = getattr(self.runner, "status", None)
        if status is None:
            return
        if not status.is_cuda:
            code = int(status[0])
        if code:
            self.runner.raise_on_status(code)

    def _settle(self, out: StepOutput) -> None:
        """Resolve the step in flight, if there is one."""
        if self._inflight is not None:
            plan, pending = self._inflight
            self._inflight = None
            self._resolve(plan, pending, out)

    def _fail(self, exc: Exception, out: StepOutput) -> StepOutput:
        """A step failed (the step function raised, or a kernel left a status): every request in
        flight ends with ``error`` and gives back what it holds; the engine goes on serving.
        After ``max_step_failures`` failures in a row the error is passed on."""
        self.last_error = f"{type(exc).__name__}: {exc}"
        self.stats.failed_steps += 1
        self._failures_in_a_row += 1
        self._inflight = None
        self.scheduler.fail_all()
        out.finished = self._drain()
        if self._failures_in_a_row >= self.max_step_failures:
            raise exc
        return out

    def step(self) -> StepOutput:
        out = StepOutput()
        try:
            return self._step(out)
        except Exception as exc:
            return self._fail(exc, out)

    def _step(self, out: StepOutput) -> StepOutput:
        t0 = time.perf_counter()
        if self._inflight is not None and not self._can_run_ahead():
            self._settle(out)
        plan = self.scheduler.schedule()
        t1 = time.perf_counter()
        out.preempted = len(plan.preempted)
        self.stats.preemptions += out.preempted
        self.stats.schedule_ms += (t1 - t0) * 1e3
        if plan.is_empty():
            self._settle(out)
            out.finished = self._drain()
            return out
        out.did_work = True
        out.num_tokens = plan.num_tokens
        logits = self.step_fn(plan)
        t2 = time.perf_counter()
        rows = [(self.scheduler.seqs[s].params, self.states[s]) for s in plan.sampled_seqs]
        ahead = (self.run_ahead and not self._needs_host and logits is not None and logits.is_cuda
                 and bool(rows))
        block = getattr(self.runner, "status_and_sampled", None)
        if not rows:
            pending = PendingSample(0, tokens=[])
        elif ahead:
            pending = self.sampler.launch(logits, rows, self.runner.sampled, block)
        else:
            self._settle(out)        # the host needs this step's logits: nothing may be ahead of it
            on_device = logits is not None and logits.is_cuda and block is not None
            toks = self.sampler.sample(logits, rows, self.runner.sampled if on_device else None,
                                       block if on_device else None)
            pending = PendingSample(len(rows), tokens=toks, status=self.sampler.last_status if on_device else 0)
            for sid, lp in zip(plan.sampled_seqs, self.sampler.last_logprobs):
                if lp is not None and sid in self._logprobs:
                    self._logprobs[sid].append(lp)
        self.scheduler.advance(plan)
        t3 = time.perf_counter()
        if self._inflight is not None:
            self.stats.ahead_steps += 1
        self._settle(out)
        if ahead:
            self._inflight = (plan, pending)
        else:
            self._resolve(plan, pending, out)
        self._failures_in_a_row = 0
        t4 = time.perf_counter()
        st = self.stats
        st.steps += 1
        st.tokens_in += plan.num_tokens
        st.forward_ms += (t2 - t1) * 1e3
        st.sample_ms += (t3 - t2) * 1e3
        st.commit_ms += (t4 - t3) * 1e3
        out.finished = self._drain()
        return out

    def _drain(self) -> List[Finished]:
        done = []
        for seq in self.scheduler.drain_finished():
            self.states.pop(seq.seq_id, None)
            self._needs_host.discard(seq.seq_id)
            lps = self._logprobs.pop(seq.seq_id, None)
            gen = seq.generated
            done.append(Finished(seq.request_id, seq.prompt_len, gen, seq.finish_reason, seq.preemptions,
                                 lps[:len(gen)] if lps is not None else None))
        return done

    # ---- run to completion ---------------------------------------------------------------
    def run(self, on_token: Optional[Callable[[object, int], None]] = None) -> List[Finished]:
        """Step until nothing is left; returns the finished requests in finishing order."""
        done: List[Finished] = []
        idle_steps = 0
        while not self.is_idle():
            out = self.step()
            if on_token:
                for rid, tok in out.new_tokens.items():
                    on_token(rid, tok)
            done += out.finished
            idle_steps = 0 if (out.did_work or out.finished) else idle_steps + 1
            if idle_steps > 2:
                raise RuntimeError("the scheduler makes no progress: a waiting request can never be started "
                                   "(cache too small for it)")
        return done
