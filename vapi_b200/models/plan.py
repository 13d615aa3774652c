"""A model as data: parts, their tensor names, and the order in which layers run."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..parts.base import Norm, Part, PositionEncoding, TensorSpec
from ..parts.embedding import OutputHead, TokenEmbedding


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes ``ModelPlan.layers`` (a layer may be named more than once: its weights
    are shared, each call site has a cache of its own).  ``cache_of`` = k makes this call
    site read the cache that call site k owns instead of having one (k < this index, and
    that site's mixer must want the same kind of cache).
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelPlan:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: TokenEmbedding
    layers: List[Part]                 # blocks
    layer_prefixes: List[str]          # checkpoint prefix of each block, e.g. "model.layers.3."
    order: List[LayerCall]
    final_norm: Norm
    final_norm_prefix: str
    head: OutputHead
    position_encodings: List[PositionEncoding] = field(default_factory=list)
    eos_token_ids: Tuple[int, ...] = ()
    config: Any = None

    def __post_init__(self) -> None:
        if len(self.layers) != len(self.layer_prefixes):
            raise ValueError("one checkpoint prefix per layer is needed")
        for i, c in enumerate(self.order):
            if not 0 <= c.layer < len(self.layers):
                raise ValueError(f"run order entry {i} names layer {c.layer} of {len(self.layers)}")
            if c.cache_of is not None:
                if not 0 <= c.cache_of < i or self.order[c.cache_of].cache_of is not None:
                    raise ValueError(f"run order entry {i}: cache_of must name an earlier entry that owns its cache")
                a = self.layers[c.layer].mixer.cache_spec()
                b = self.layers[self.order[c.cache_of].layer].mixer.cache_spec()
                if a != b:
                    raise ValueError(f"run order entry {i} cannot read the cache of entry {c.cache_of}: {a} != {b}")

    # ---- tensors -------------------------------------------------------------------
    def tensor_specs(self) -> List[TensorSpec]:
        specs: List[TensorSpec] = list(self.embedding.tensor_specs(""))
        for blk, pre in zip(self.layers, self.layer_prefixes):
            specs += blk.tensor_specs(pre)
        specs += self.final_norm.tensor_specs(self.final_norm_prefix)
        specs += self.head.tensor_specs("")
        for pe in self.position_encodings:
            specs += pe.tensor_specs("")
        seen: Dict[str, TensorSpec] = {}
        for s in specs:
            if s.name in seen and seen[s.name].shape != s.shape:
                raise ValueError(f"tensor `{s.name}` is wanted with two shapes")
            seen[s.name] = s
        return list(seen.values())

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype) -> None:
        self.embedding.bind(tensors, "", dtype)
        for blk, pre in zip(self.layers, self.layer_prefixes):
            blk.bind(tensors, pre, dtype)
        self.final_norm.bind(tensors, self.final_norm_prefix, dtype)
        self.head.bind(tensors, "", dtype)
        for pe in self.position_encodings:
            pe.bind(tensors, "", dtype)

    # ---- caches --------------------------------------------------------------------
    def cache_sites(self) -> List[Tuple[int, object]]:
        """(index in the run order, spec) of every call site that owns a cache."""
        out = []
        for i, c in enumerate(self.order):
            if c.cache_of is None:
                spec = self.layers[c.layer].mixer.cache_spec()
                if spec is not None:
                    out.append((i, spec))
        return out
