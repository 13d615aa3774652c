"""The gated short convolution mixer with a fixed-size state per request."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from .. import ops
from .base import CacheView, Mixer, StateSpec, StreamState, TensorSpec, register_mixer


class ShortConv(Mixer):
    """``in_proj`` -> B, C, x; ``g = B * x``; causal depthwise conv of length ``kernel``;
    ``y = C * conv``; ``out_proj`` (crates/vapi-backend-candle/src/models/lfm2.rs:7-13,
    438-485, 509-565).  ``bias`` switches the in_proj, conv and out_proj biases on together,
    as the reference's ``conv_bias`` does (lfm2.rs:441-464).

    Where the reference stores g for every token in paged rows, this part keeps only what
    the convolution can still reach: the last ``kernel - 1`` rows of g, a state of fixed size
    in the request's slot.
    """

    def __init__(self, hidden: int, kernel: int, bias: bool = False,
                 names: Optional[Dict[str, str]] = None):
        if not 1 <= kernel <= 8:
            raise ValueError(f"conv kernel length {kernel} is outside 1..8")
        self.hidden, self.kernel, self.bias = int(hidden), int(kernel), bool(bias)
        self.names = {"in": "in_proj", "conv": "conv", "out": "out_proj"}
        if names:
            self.names.update(names)
        self.w_in = self.b_in = self.taps = self.b_conv = self.w_out = self.b_out = None

    def cache_spec(self):
        if self.kernel == 1:
            return None
        return StateSpec("shortconv", (self.kernel - 1, self.hidden))

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        n, h, L = self.names, self.hidden, self.kernel
        specs = [TensorSpec(f"{prefix}{n['in']}.weight", (3 * h, h)),
                 TensorSpec(f"{prefix}{n['conv']}.weight", (h, 1, L), role="vector"),
                 TensorSpec(f"{prefix}{n['out']}.weight", (h, h))]
        if self.bias:
            specs += [TensorSpec(f"{prefix}{n['in']}.bias", (3 * h,), role="vector"),
                      TensorSpec(f"{prefix}{n['conv']}.bias", (h,), role="vector"),
                      TensorSpec(f"{prefix}{n['out']}.bias", (h,), role="vector")]
        return specs

    def bind(self, tensors, prefix, dtype):
        n = self.names
        self.w_in = tensors[f"{prefix}{n['in']}.weight"].contiguous()
        self.w_out = tensors[f"{prefix}{n['out']}.weight"].contiguous()
        # (H, 1, L) -> (L, H): one row of channel weights per tap, oldest first
        self.taps = tensors[f"{prefix}{n['conv']}.weight"].squeeze(1).t().contiguous()
        if self.bias:
            self.b_in = tensors[f"{prefix}{n['in']}.bias"].contiguous()
            self.b_conv = tensors[f"{prefix}{n['conv']}.bias"].contiguous()
            self.b_out = tensors[f"{prefix}{n['out']}.bias"].contiguous()

    def forward(self, a: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        h3 = ops.linear(a, self.w_in)          # the in_proj bias is applied inside the kernel
        y = ops.shortconv(h3, self.b_in, self.taps, self.b_conv, cache.tensor, ctx.state_slots,
                          ctx.tok_seq, ctx.cu_q, ctx.positions, ctx.status)
        return ops.linear(y, self.w_out, self.b_out)

    def forward_stream(self, a, ctx, cache, x, next_weight):
        n = x.shape[0]
        if not (ops.few_rows_applies(n, self.w_in) and ops.few_rows_applies(n, self.w_out)):
            return NotImplemented
        if ctx.max_q == 1 and ctx.n == ctx.num_seqs and ops.skinny_shortconv_applies(n, self.w_in, self.kernel, cache.tensor):
            # a decode step: every token is a sequence of its own, and the gated convolution rides
            # on in_proj as its epilogue
            y = ops.skinny_shortconv(self.w_in, xw=a.xw, ss_in=a.ss, eps=a.eps, in_bias=self.b_in, taps=self.taps,
                                     conv_bias=self.b_conv, state_layer=cache.tensor, state_slots=ctx.state_slots,
                                     positions=ctx.positions, status=ctx.status)
        else:
            h3 = ops.few_rows_linear(self.w_in, xw=a.xw, ss_in=a.ss, eps=a.eps, epilogue="bf16")
            y = ops.shortconv(h3, self.b_in, self.taps, self.b_conv, cache.tensor, ctx.state_slots,
                              ctx.tok_seq, ctx.cu_q, ctx.positions, ctx.status)
        ss, xw = ops.few_rows_linear(self.w_out, act=y, epilogue="resid", resid=x, bias=self.b_out, next_weight=next_weight)
        return StreamState(xw, ss)


register_mixer("shortconv", ShortConv)
