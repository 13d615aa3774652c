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
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..sampling.params import FinishReason, SamplingParams
from ..sampling.sampler import Sampler, SamplerState
from .runner import ModelRunner
from .scheduler import AdmitError, Scheduler, SchedulerConfig, SeqStatus, StepPlan


@dataclass
class Finished:
    request_id: object
    prompt_tokens: int
    tokens: List[int]
    reason: FinishReason
    preemptions: int = 0


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
    schedule_ms: float = 0.0
    forward_ms: float = 0.0
    sample_ms: float = 0.0
    commit_ms: float = 0.0


class Engine:
    def __init__(self, runner: ModelRunner, cfg: Optional[SchedulerConfig] = None, *,
                 max_step_failures: int = 3, use_graphs: bool = True):
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
        return sid

    def cancel(self, sid: int) -> None:
        self.scheduler.cancel(sid)

    def is_idle(self) -> bool:
        return self.scheduler.is_idle() and not self.scheduler.finished

    # ---- one step ---------------------------------------------------------------------
    def _run(self, plan: StepPlan) -> Optional[torch.Tensor]:
        if self.use_graphs and plan.pure_decode and hasattr(self.runner, "step_decode_graph"):
            out = self.runner.step_decode_graph(None, plan=plan)
            if out is not None:
                return out
        return self.runner.step(None, plan=plan)

    def step(self) -> StepOutput:
        out = StepOutput()
        t0 = time.perf_counter()
        plan = self.scheduler.schedule()
        t1 = time.perf_counter()
        out.preempted = len(plan.preempted)
        self.stats.preemptions += out.preempted
        self.stats.schedule_ms += (t1 - t0) * 1e3
        if plan.is_empty():
            out.finished = self._drain()
            return out
        out.did_work = True
        out.num_tokens = plan.num_tokens
        try:
            logits = self.step_fn(plan)
            t2 = time.perf_counter()
            sampled: List[int] = []
            if plan.sampled_seqs:
                rows = [(self.scheduler.seqs[s].params, self.states[s]) for s in plan.sampled_seqs]
                sampled = self.sampler.sample(logits, rows)
            t3 = time.perf_counter()
        except Exception as exc:
            self.last_error = f"{type(exc).__name__}: {exc}"
            self.stats.failed_steps += 1
            self._failures_in_a_row += 1
            self.scheduler.fail_all()
            out.finished = self._drain()
            if self._failures_in_a_row >= self.max_step_failures:
                raise
            return out
        self._failures_in_a_row = 0
        for sid, tok in zip(plan.sampled_seqs, sampled):
            self.states[sid].observe(tok)
            out.new_tokens[self.scheduler.seqs[sid].request_id] = tok
        self.scheduler.commit(plan, sampled)
        t4 = time.perf_counter()
        st = self.stats
        st.steps += 1
        st.tokens_in += plan.num_tokens
        st.tokens_out += len(sampled)
        st.forward_ms += (t2 - t1) * 1e3
        st.sample_ms += (t3 - t2) * 1e3
        st.commit_ms += (t4 - t3) * 1e3
        out.finished = self._drain()
        return out

    def _drain(self) -> List[Finished]:
        done = []
        for seq in self.scheduler.drain_finished():
            self.states.pop(seq.seq_id, None)
            done.append(Finished(seq.request_id, seq.prompt_len, seq.generated, seq.finish_reason, seq.preemptions))
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
