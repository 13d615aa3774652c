"""Run-time configuration: a TOML file with the reference's sections and key names.

Only the keys that concern an engine on one GPU exist; each has the reference's name,
meaning and default (crates/vapi-core/src/config.rs:137-300).  Unknown sections or keys are
errors, as with the reference's ``deny_unknown_fields``.  Precedence of the file:
``--config`` flag > ``$VAPI_CONFIG`` > ``./vapi.toml`` > defaults
(crates/vapi-core/src/cli.rs:26-56).

    [model]
    path = "/models/lfm2"      # folder with config.json and safetensors
    dtype = "auto"             # auto | bf16 | f32   (auto = bf16 on CUDA)
    device = "auto"            # auto | cuda
    max_context = 8192
    kv_cache_fraction = 0.85   # of free device memory, when num_blocks is not given
    num_blocks = 2048          # cache pages; the reference's name for them
    cuda_graphs = false

    [worker]
    max_concurrent_seqs = 64
    max_batched_tokens = 8192
    prefill_chunk_tokens = 2048
    max_step_failures = 3

    [cache]
    watermark = 0.01
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, Optional


class RuntimeConfigError(ValueError):
    pass


@dataclass
class ModelSection:
    path: Optional[str] = None
    dtype: str = "auto"
    device: str = "auto"
    max_context: int = 8192
    kv_cache_fraction: float = 0.85
    num_blocks: Optional[int] = None
    cuda_graphs: bool = False


@dataclass
class WorkerSection:
    max_concurrent_seqs: int = 64
    max_batched_tokens: int = 8192
    prefill_chunk_tokens: int = 2048
    max_step_failures: int = 3


@dataclass
class CacheSection:
    watermark: float = 0.01


@dataclass
class RuntimeConfig:
    model: ModelSection = field(default_factory=ModelSection)
    worker: WorkerSection = field(default_factory=WorkerSection)
    cache: CacheSection = field(default_factory=CacheSection)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RuntimeConfig":
        cfg = cls()
        sections = {"model": cfg.model, "worker": cfg.worker, "cache": cfg.cache}
        for sec, body in d.items():
            if sec not in sections:
                raise RuntimeConfigError(f"unknown section [{sec}]; known: {sorted(sections)}")
            if not isinstance(body, dict):
                raise RuntimeConfigError(f"[{sec}] must be a table")
            known = {f.name: f for f in fields(sections[sec])}
            for k, v in body.items():
                if k not in known:
                    raise RuntimeConfigError(f"unknown key `{k}` in [{sec}]; known: {sorted(known)}")
                setattr(sections[sec], k, v)
        cfg.validate()
        return cfg

    @classmethod
    def load(cls, path: Optional[str] = None) -> "RuntimeConfig":
        """``path`` > ``$VAPI_CONFIG`` > ``./vapi.toml`` > defaults."""
        import tomllib
        cand = path or os.environ.get("VAPI_CONFIG")
        if cand is None and os.path.isfile("vapi.toml"):
            cand = "vapi.toml"
        if cand is None:
            return cls()
        if not os.path.isfile(cand):
            raise RuntimeConfigError(f"config file {cand} does not exist")
        with open(cand, "rb") as f:
            return cls.from_dict(tomllib.load(f))

    def validate(self) -> None:
        m, w, c = self.model, self.worker, self.cache
        if m.dtype not in ("auto", "bf16", "bfloat16", "f32", "float32"):
            raise RuntimeConfigError(f"model.dtype `{m.dtype}` is not one of auto, bf16, f32")
        if m.device not in ("auto", "cuda"):
            raise RuntimeConfigError(f"model.device `{m.device}`: this engine runs on CUDA only")
        if not 0.0 < float(m.kv_cache_fraction) <= 1.0:
            raise RuntimeConfigError("model.kv_cache_fraction must be in (0, 1]")
        if m.num_blocks is not None and int(m.num_blocks) <= 0:
            raise RuntimeConfigError("model.num_blocks must be positive")
        for name in ("max_concurrent_seqs", "max_batched_tokens", "prefill_chunk_tokens", "max_step_failures"):
            if int(getattr(w, name)) <= 0:
                raise RuntimeConfigError(f"worker.{name} must be positive")
        if int(m.max_context) <= 1:
            raise RuntimeConfigError("model.max_context must be at least 2")
        if not 0.0 <= float(c.watermark) < 1.0:
            raise RuntimeConfigError("cache.watermark must be in [0, 1)")

    def resolved_dtype(self) -> str:
        return "float32" if self.model.dtype in ("f32", "float32") else "bfloat16"
