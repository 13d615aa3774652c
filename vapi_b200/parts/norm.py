"""RMSNorm with the residual add folded in."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .base import Norm, NormedStream, TensorSpec, register_norm


class RMSNorm(Norm):
    """``y = x * rsqrt(mean(x^2) + eps) * w``: the weight multiplies as it is (no ``1 + w``)
    (crates/vapi-backend-candle/src/models/lfm2.rs:626-628).  Mean, rsqrt and the residual
    sum are float32 whatever the activation dtype."""

    def __init__(self, dim: int, eps: float, weight_name: str = "weight"):
        self.dim, self.eps, self.weight_name = int(dim), float(eps), weight_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(f"{prefix}{self.weight_name}", (self.dim,), role="vector", init="ones")]

    def bind(self, tensors: Dict[str, torch.Tensor], prefix: str, dtype: torch.dtype) -> None:
        self.weight = tensors[f"{prefix}{self.weight_name}"].contiguous()

    def apply(self, x, delta, dtype, rows=None):
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, dtype, rows)

    def stream_weight(self):
        return self.weight

    def deferred(self, state):
        return NormedStream(state.xw, state.ss, self.eps)


register_norm("rmsnorm", RMSNorm)
