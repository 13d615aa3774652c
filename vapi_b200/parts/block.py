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


register_block("prenorm", PreNormBlock)
