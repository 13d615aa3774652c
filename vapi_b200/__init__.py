"""vapi_b200: a small, whole LFM2 inference engine for one B200.

From a model folder (config.json + safetensors, or seeded random weights) to generated
tokens: typed configuration and architecture registry, weights by name, layers assembled
from parts, a paged cache with per-request state slots, one step function for mixed
batches, a continuous-batching scheduler, sampling, and hand-written sm_100a kernels.
"""
from .sampling.params import FinishReason, SamplingParams

__version__ = "0.1.0"


def __getattr__(name):
    # the heavy parts import torch and (on first use) build kernels: load them lazily
    if name in ("LLM", "generate", "Completion"):
        from . import api
        return getattr(api, name)
    if name == "ModelRunner":
        from .engine.runner import ModelRunner
        return ModelRunner
    if name == "RuntimeConfig":
        from .config.runtime import RuntimeConfig
        return RuntimeConfig
    raise AttributeError(name)


__all__ = ["LLM", "generate", "Completion", "SamplingParams", "FinishReason", "ModelRunner", "RuntimeConfig"]
