"""The arrangement of parts in a layer."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch

from .base import CacheView, FeedForward, Mixer, Norm, Part, StreamState, TensorSpec

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

    def first_norm(self) -> Norm:
        """The norm that reads the stream first in this block (its producer works for it)."""
        return self.mixer_norm

    def forward_stream(self, x: torch.Tensor, state: StreamState, ctx: Any, cache: CacheView,
                       next_weight: torch.Tensor) -> StreamState:
        """The same block for steps of a few rows: a norm is not run but handed, as a
        description, to its consumer's first product; each part's last product adds into ``x``
        and leaves the :class:`StreamState` the following norm needs (``next_weight`` is the
        weight of the norm that reads the stream after this block).  A part without a stream
        form is run the ordinary way between two small kernels."""
        from .. import ops
        mid_weight = self.ffn_norm.stream_weight()
        a = self.mixer_norm.deferred(state) if state is not None else None
        out = self.mixer.forward_stream(a, ctx, cache, x, mid_weight) if (a is not None and mid_weight is not None) else NotImplemented
        if out is NotImplemented:
            delta = self.mixer.forward(self.mixer_norm.apply(x, None, ctx.dtype), ctx, cache)
            out = self._add(ops, x, delta, mid_weight)
        f = self.ffn_norm.deferred(out) if out is not None else None
        out2 = self.ffn.forward_stream(f, ctx, x, next_weight) if (f is not None and next_weight is not None) else NotImplemented
        if out2 is NotImplemented:
            delta = self.ffn.forward(self.ffn_norm.apply(x, None, ctx.dtype), ctx)
            out2 = self._add(ops, x, delta, next_weight)
        return out2

    @staticmethod
    def _add(ops, x, delta, weight):
        if weight is None:
            ops.add_residual(x, delta)
            return None
        ss, xw = ops.add_residual_ss(x, delta, weight)
        return StreamState(xw, ss)


register_block("prenorm", PreNormBlock)
