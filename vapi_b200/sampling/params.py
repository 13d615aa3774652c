"""Sampling options of a request: names, defaults and limits of the reference
(crates/vapi-core/src/sampling.rs:11-58, 84-116, 134-176)."""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Optional, Tuple

F32_EPSILON = 1.1920929e-07


class FinishReason(str, enum.Enum):
    STOP = "stop"             # an EOS token or a stop token id
    LENGTH = "length"         # max_tokens or the context limit
    CANCELLED = "cancelled"
    ERROR = "error"


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: Optional[int] = None
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    max_tokens: int = 256
    n: int = 1                          # completions per prompt (each an independent request here)
    seed: Optional[int] = None
    logprobs: Optional[int] = None      # report the chosen token's log-probability and this many top ones
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False

    def validate(self) -> None:
        if not 0.0 <= self.temperature <= 2.0:
            raise ValueError("temperature must be in [0, 2]")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError("min_p must be in [0, 1]")
        if self.top_k is not None and self.top_k < 1:
            raise ValueError("top_k must be >= 1")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if not 1 <= self.n <= 8:
            raise ValueError("n must be in [1, 8]")
        if self.repetition_penalty <= 0.0:
            raise ValueError("repetition_penalty must be > 0")
        if self.logprobs is not None and not 0 <= self.logprobs <= 20:
            raise ValueError("logprobs must be <= 20")

    @property
    def is_greedy(self) -> bool:
        """Greedy decoding: take the argmax and never touch a random generator."""
        return self.temperature <= F32_EPSILON

    @property
    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0

    @property
    def device_drawable(self) -> bool:
        """Nothing but temperature (and penalties): a Gumbel-max draw on the device samples
        it exactly (crates/vapi-engine/src/sampler.rs:45-47)."""
        return (not self.is_greedy) and self.top_k is None and self.top_p >= 1.0 and self.min_p <= 0.0

    @property
    def inv_temperature(self) -> float:
        return 1.0 if self.is_greedy else 1.0 / max(self.temperature, 1e-5)
