"""The arrangement of parts in a layer."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch

from .base import CacheView, FeedForward, Mixer, Norm, Part, TensorSpec

BLOCKS: Dict[str, Callable[..., "Part"]] = {}


def register_block(name: str, ctor: Callable[..., "Part"], *, replace: bool = False) -> None:
    if name in BLOCKS and not replace and BLOCKS[name] is not ctor:
        raise ValueError(f"block `{name}` is already registered")
    BLOCKS[name] = ctor


class PreNormBlock(Part):
    """``x <- x + mixer(norm_m(x))``; ``x <- x + ffn(norm_f(x))``
    (crates/vapi-backend-candle/src/models/lfm2.rs:633-648).

    The residual stream ``x`` is float32.  A layer's output is not added right away: it is
    handed on as ``delta`` and the next norm adds it while it reads the row, so each add
    costs no pass of its own.  ``forward`` therefore takes the pending delta of the layer
    before and returns its own.

    ``sub`` gives the checkpoint sub-prefix of each part, e.g. ``{"mixer": "conv.",
    "mixer_norm": "operator_norm.", "ffn": "feed_forward.", "ffn_norm": "ffn_norm."}``.
    """

    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward,
                 sub: Dict[str, str]):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, self.sub = mixer_norm, mixer, ffn_norm, ffn, dict(sub)

    def _parts(self):
        return (("mixer_norm", self.mixer_norm), ("mixer", self.mixer),
                ("ffn_norm", self.ffn_norm), ("ffn", self.ffn))

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        out: List[TensorSpec] = []
        for key, part in self._parts():
            out += part.tensor_specs(prefix + self.sub[key])
        return out

    def bind(self, tensors, prefix, dtype):
        for key, part in self._parts():
            part.bind(tensors, prefix + self.sub[key], dtype)

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], ctx: Any,
                cache: CacheView) -> torch.Tensor:
        a = self.mixer_norm.apply(x, delta, ctx.dtype)
        d1 = self.mixer.forward(a, ctx, cache)
        f = self.ffn_norm.apply(x, d1, ctx.dtype)
        return self.ffn.forward(f, ctx)

    def forward_stream(self, x: torch.Tensor, ss: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        """The same block for steps of a few rows: norms are applied inside their consumer's
        first product, results are added into ``x`` by the last product of each part, and the
        partial sums of squares of ``x`` travel from producer to consumer as ``ss``.  A part
        without a stream form is run the ordinary way between two small kernels."""
        from .. import ops
        a = self.mixer_norm.deferred(x, ss)
        out = self.mixer.forward_stream(a, ctx, cache, x) if a is not None else NotImplemented
        if out is NotImplemented:
            delta = self.mixer.forward(self.mixer_norm.apply(x, None, ctx.dtype), ctx, cache)
            out = ops.add_residual_ss(x, delta)
        f = self.ffn_norm.deferred(x, out)
        out2 = self.ffn.forward_stream(f, ctx, x) if f is not None else NotImplemented
        if out2 is NotImplemented:
            delta = self.ffn.forward(self.ffn_norm.apply(x, None, ctx.dtype), ctx)
            out2 = ops.add_residual_ss(x, delta)
        return out2


register_block("prenorm", PreNormBlock)
