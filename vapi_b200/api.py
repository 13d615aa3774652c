"""The Python entry point: load a model folder, generate tokens.

    from vapi_b200 import LLM, SamplingParams
    llm = LLM("/models/lfm2", dtype="bf16", num_blocks=2048)
    out = llm.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.0, max_tokens=16))

Token ids in, token ids out: text (tokenizer, chat template, detokenizer) is outside this
engine.  Options carry the reference's names (``[model]`` / ``[worker]`` / ``[cache]`` keys
of its TOML, crates/vapi-core/src/config.rs:137-300; sampling fields of
crates/vapi-core/src/sampling.rs:11-58).  The reference has no Python API; the nearest
programmatic entry is its decode_profile example
(crates/vapi-backend-candle/examples/decode_profile.rs:21-28).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, List, Optional, Sequence, Union

from .config.runtime import RuntimeConfig
from .engine.engine import Engine
from .engine.runner import ModelRunner
from .engine.scheduler import SchedulerConfig
from .sampling.params import SamplingParams


@dataclass
class Completion:
    request_id: object
    prompt_tokens: int
    tokens: List[int]
    finish_reason: str
    preemptions: int = 0
    index: int = 0                      # which of the prompt's ``n`` completions this is
    logprobs: Optional[list] = None     # per generated token: sampling.sampler.TokenLogprobs, when asked for


class LLM:
    """A loaded model with its cache and scheduler on ``cuda:0``."""

    def __init__(self, model: Optional[str] = None, *, dtype: str = "auto", device: str = "cuda",
                 max_context: int = 8192, kv_cache_fraction: float = 0.85, num_blocks: Optional[int] = None,
                 cuda_graphs: bool = True, max_concurrent_seqs: int = 64, max_batched_tokens: int = 8192,
                 prefill_chunk_tokens: int = 2048, watermark: float = 0.01, max_step_failures: int = 3,
                 random_weights: Optional[int] = None, config_json: Optional[Dict[str, Any]] = None,
                 page_size: Optional[int] = None, validate: bool = False, run_ahead: Optional[bool] = None):
        dt = "float32" if str(dtype).lower() in ("f32", "fp32", "float32") else "bfloat16"
        kw = dict(dtype=dt, device=device, page_size=page_size or ModelRunner.default_page_size,
                  num_pages=num_blocks, max_requests=max_concurrent_seqs,
                  max_batched_tokens=max_batched_tokens, max_context=max_context, watermark=watermark,
                  kv_cache_fraction=kv_cache_fraction, validate=validate)
        if random_weights is not None:
            if config_json is None:
                raise ValueError("random weights need a config_json (the architecture's config.json keys)")
            self.runner = ModelRunner.from_random(config_json, int(random_weights), **kw)
        else:
            if model is None:
                raise ValueError("give a model folder, or random_weights with config_json")
            self.runner = ModelRunner.from_dir(model, **kw)
        self.engine = Engine(self.runner, SchedulerConfig(
            max_concurrent_seqs=max_concurrent_seqs, max_batched_tokens=max_batched_tokens,
            prefill_chunk_tokens=prefill_chunk_tokens, max_context=max_context),
            max_step_failures=max_step_failures, use_graphs=cuda_graphs, run_ahead=run_ahead)
        self._next = 0

    @classmethod
    def from_config(cls, cfg: RuntimeConfig, **overrides: Any) -> "LLM":
        m, w, c = cfg.model, cfg.worker, cfg.cache
        kw = dict(model=m.path, dtype=cfg.resolved_dtype(), max_context=m.max_context,
                  kv_cache_fraction=m.kv_cache_fraction, num_blocks=m.num_blocks, cuda_graphs=m.cuda_graphs,
                  max_concurrent_seqs=w.max_concurrent_seqs, max_batched_tokens=w.max_batched_tokens,
                  prefill_chunk_tokens=w.prefill_chunk_tokens, watermark=c.watermark,
                  max_step_failures=w.max_step_failures)
        kw.update(overrides)
        return cls(**kw)

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 on_token=None, raise_on_error: bool = True) -> List[Completion]:
        """Generate for every prompt (lists of token ids) with continuous batching; results
        come back in the order of ``prompts``.  With ``n`` above 1 a prompt gets that many
        completions, one after the other in the result (``Completion.index`` says which); each is
        a request of its own, seeded ``seed + index`` when a seed is given.  (The reference forks
        them from one prefill through its prefix cache, which this engine does not have.)

        A step that fails ends the requests in flight with the finish reason ``"error"`` and leaves
        the engine usable, as in the reference; this call then raises with the step's message,
        unless ``raise_on_error`` is false, in which case those completions come back as they are."""
        if params is None:
            params = SamplingParams()
        plist = [params] * len(prompts) if isinstance(params, SamplingParams) else list(params)
        if len(plist) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        ids = []
        for prompt, p in zip(prompts, plist):
            p.validate()
            for i in range(p.n):
                rid = self._next
                self._next += 1
                one = p if p.n == 1 else replace(p, n=1, seed=None if p.seed is None else p.seed + i)
                self.engine.admit(rid, prompt, one)
                ids.append((rid, i))
        done = {f.request_id: f for f in self.engine.run(on_token)}
        out = []
        for rid, i in ids:
            f = done[rid]
            out.append(Completion(rid, f.prompt_tokens, f.tokens, f.reason.value, f.preemptions, i, f.logprobs))
        if raise_on_error and any(c.finish_reason == "error" for c in out):
            failed = sum(c.finish_reason == "error" for c in out)
            raise RuntimeError(f"{failed} of {len(out)} requests ended in a failed step: {self.engine.last_error}")
        return out


def generate(model: str, prompts: Sequence[Sequence[int]], *, max_tokens: int = 256, temperature: float = 0.0,
             seed: Optional[int] = None, stop_token_ids: Sequence[int] = (), **llm_options: Any) -> List[List[int]]:
    """One call from a model folder to generated token ids (greedy by default)."""
    llm = LLM(model, **llm_options)
    p = SamplingParams(temperature=temperature, max_tokens=max_tokens, seed=seed,
                       stop_token_ids=tuple(int(t) for t in stop_token_ids))
    return [c.tokens for c in llm.generate(prompts, p)]
