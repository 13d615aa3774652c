"""Token embedding and the output head."""
from __future__ import annotations

from typing import Any, List, Optional

import torch

from .. import ops
from .base import Part, TensorSpec


class TokenEmbedding(Part):
    """Row gather from a [vocab, hidden] table, no scaling
    (crates/vapi-backend-candle/src/models/lfm2.rs:675, 808).  Starts the float32 stream."""

    def __init__(self, vocab: int, hidden: int, name: str = "model.embed_tokens.weight"):
        self.vocab, self.hidden, self.name = int(vocab), int(hidden), name
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str = "") -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab, self.hidden))]

    def bind(self, tensors, prefix, dtype):
        self.table = tensors[self.name].contiguous()

    def forward(self, ctx: Any, next_weight: Optional[torch.Tensor] = None):
        """The stream; with ``next_weight`` also what a deferred norm needs: ``(x, ss, xw)``."""
        return ops.embed(self.table, ctx.tokens, ctx.status, next_weight)


class OutputHead(Part):
    """Logits in float32 for the wanted rows: ``norm(x)[rows] @ W.T``.

    ``tied`` (or a checkpoint without the head's tensor) reuses the embedding table
    (crates/vapi-backend-candle/src/models/lfm2.rs:676-680, 803-818)."""

    def __init__(self, vocab: int, hidden: int, tied: bool, embedding: TokenEmbedding,
                 name: str = "lm_head.weight"):
        self.vocab, self.hidden, self.tied, self.embedding, self.name = int(vocab), int(hidden), bool(tied), embedding, name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str = "") -> List[TensorSpec]:
        if self.tied:
            return []
        # optional: a checkpoint that leaves it out falls back to the embedding table
        return [TensorSpec(self.name, (self.vocab, self.hidden), optional=True)]

    def bind(self, tensors, prefix, dtype):
        w = None if self.tied else tensors.get(self.name)
        self.weight = (w if w is not None else tensors[self.embedding.name]).contiguous()

    def forward(self, xn: torch.Tensor) -> torch.Tensor:
        return ops.linear(xn, self.weight, None, torch.float32)

    def forward_stream(self, a):
        """Logits of every row of a lazily normed stream (decode steps), or NotImplemented."""
        if not ops.few_rows_applies(a.xw.shape[0], self.weight):
            return NotImplemented
        return ops.few_rows_linear(self.weight, xw=a.xw, ss_in=a.ss, eps=a.eps, epilogue="f32")
