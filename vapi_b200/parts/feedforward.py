"""Dense SwiGLU feed-forward."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from .. import ops
from .base import FeedForward, StreamState, TensorSpec, register_feed_forward


class SwiGLU(FeedForward):
    """``down( silu(gate f) * (up f) )`` without biases; gate and up are stacked into one
    matrix at bind time so they are one product
    (crates/vapi-backend-candle/src/models/lfm2.rs:568-595).  ``names`` maps gate/up/down to
    the checkpoint's sub-names (LFM2: w1 / w3 / w2)."""

    def __init__(self, hidden: int, ff: int, names: Optional[Dict[str, str]] = None):
        self.hidden, self.ff = int(hidden), int(ff)
        self.names = {"gate": "w1", "up": "w3", "down": "w2"}
        if names:
            self.names.update(names)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        n = self.names
        return [TensorSpec(f"{prefix}{n['gate']}.weight", (self.ff, self.hidden)),
                TensorSpec(f"{prefix}{n['up']}.weight", (self.ff, self.hidden)),
                TensorSpec(f"{prefix}{n['down']}.weight", (self.hidden, self.ff))]

    def bind(self, tensors, prefix, dtype):
        n = self.names
        g, u = tensors[f"{prefix}{n['gate']}.weight"], tensors[f"{prefix}{n['up']}.weight"]
        wd = g.dtype if g.dtype == u.dtype else torch.float32
        self.w_gate_up = torch.cat([g.to(wd), u.to(wd)], 0).contiguous()
        self.w_down = tensors[f"{prefix}{n['down']}.weight"].contiguous()

    def forward(self, f: torch.Tensor, ctx: Any) -> torch.Tensor:
        return ops.linear(ops.linear_swiglu(f, self.w_gate_up), self.w_down)

    def forward_stream(self, f, ctx, x, next_weight):
        n = x.shape[0]
        if not (ops.few_rows_applies(n, self.w_gate_up) and ops.few_rows_applies(n, self.w_down)):
            return NotImplemented
        s = ops.few_rows_linear(self.w_gate_up, xw=f.xw, ss_in=f.ss, eps=f.eps, epilogue="swiglu")
        ss, xw = ops.few_rows_linear(self.w_down, act=s, epilogue="resid", resid=x, next_weight=next_weight)
        return StreamState(xw, ss)


register_feed_forward("swiglu", SwiGLU)
