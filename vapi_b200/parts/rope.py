"""Rotary position encoding: per-step cos/sin rows in float32."""
from __future__ import annotations

from typing import Any, Dict, Tuple

import torch

from .. import ops
from .base import PositionEncoding, register_position_encoding


class RotaryEncoding(PositionEncoding):
    """Rotate-half RoPE over the first ``rot_dim`` elements of a head.

    ``inv_freq_i = 1 / theta^(2i / rot_dim)`` in float32, angle = position * inv_freq_i as a
    float32 product (crates/vapi-backend-candle/src/models/lfm2.rs:163-183).  The reference
    rounds its cos/sin tables to the model dtype; here they stay float32 and are computed for
    the step's positions only, so there is no table of ``max_positions`` rows to hold.
    ``prepare`` returns ``(cos, sin)`` [n, rot_dim/2] which an attention mixer applies.
    """

    def __init__(self, rot_dim: int, theta: float, max_positions: int, name: str = "rope"):
        if rot_dim <= 0 or rot_dim % 2:
            raise ValueError(f"rotary width {rot_dim} must be a positive even number")
        self.rot_dim, self.theta, self.max_positions, self.name = int(rot_dim), float(theta), int(max_positions), name
        self._inv_freq: Dict[Any, torch.Tensor] = {}

    def inv_freq(self, device: torch.device) -> torch.Tensor:
        key = str(device)
        t = self._inv_freq.get(key)
        if t is None:
            theta = torch.tensor(self.theta, dtype=torch.float32)
            expo = torch.arange(0, self.rot_dim, 2, dtype=torch.float32) / float(self.rot_dim)
            t = (1.0 / torch.pow(theta, expo)).to(device).contiguous()
            self._inv_freq[key] = t
        return t

    def prepare(self, ctx: Any) -> Tuple[torch.Tensor, torch.Tensor]:
        return ops.rope_cos_sin(ctx.positions, self.inv_freq(ctx.positions.device))


register_position_encoding("rope", RotaryEncoding)
