"""Interfaces of the parts a model is put together from.

A model is a list of blocks; a block arranges a *mixer* (attention, short convolution, or
anything else that moves information between tokens), a *feed-forward*, and *norms*; a
*position encoding* prepares per-step tensors that mixers may use.  Each part

* is constructed from plain sizes and constants (never from a model configuration object),
* names the checkpoint tensors it wants (:class:`TensorSpec`) under a prefix it is given,
* says what kind of cache it needs (:class:`PagedSpec`, :class:`StateSpec` or ``None``),
* binds its loaded tensors once (``bind``) and then runs on a step (``forward``).

No part knows which model it is in.  Parts are looked up by name in small registries so a
test (or a new architecture) can add one without touching this package's files.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

# --------------------------------------------------------------------------------------
# what a part asks of the checkpoint


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part needs.

    ``role`` decides the run-time dtype: a ``matrix`` is an operand of a matrix product or
    an embedding table and is kept in the compute dtype (bfloat16 when serving), except
    that a tensor the checkpoint stores in 32-bit stays 32-bit; a ``vector`` (norm weight,
    bias, conv tap) is always handed to kernels as float32; a ``table`` is integer data and
    becomes int32.  ``init`` is how the random-weights writer fills it.
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"      # matrix | vector | table
    init: str = "normal"      # normal | ones | zeros
    optional: bool = False


# --------------------------------------------------------------------------------------
# what a part asks of the cache manager


@dataclass(frozen=True)
class PagedBuffer:
    """One thing a mixer keeps for every token of a request: ``rows`` rows of ``width`` elements
    (keys: one row of ``head_dim`` per kv head; a latent or a conv input: one row of its width)."""

    name: str
    rows: int
    width: int


@dataclass(frozen=True)
class PagedSpec:
    """Per-token cache in pages, described so that the cache manager can lay it out without
    knowing what the mixer is: a tuple of :class:`PagedBuffer`, each holding some rows of some
    width for every token (the reference's ``LayerLayout::{Kv, Rows}``,
    crates/vapi-backend-candle/src/cache.rs:22-45).  Keys and values of grouped-query attention
    are the special case of two buffers of ``n_kv`` rows of ``head_dim`` (:meth:`kv`).

    A page holds ``page_size`` tokens; inside a page the buffers follow one another, each as
    ``[rows, page_size, width]``.  Buffers of equal shape therefore lie as
    ``[n_buffers, rows, page_size, width]`` (:meth:`CacheView.stacked`), which is what the
    attention kernels read.

    ``window`` = 0 keeps every position; ``window`` = W > 0 means positions more than W
    behind the newest are never read again, so the manager may give their pages back.
    Layers with equal specs share one group: one pool of pages, one block table a request.
    """

    buffers: Tuple[PagedBuffer, ...]
    window: int = 0

    @classmethod
    def kv(cls, n_kv: int, head_dim: int, window: int = 0) -> "PagedSpec":
        """Keys and values of ``n_kv`` heads of ``head_dim``."""
        return cls((PagedBuffer("k", int(n_kv), int(head_dim)), PagedBuffer("v", int(n_kv), int(head_dim))), int(window))

    @classmethod
    def rows(cls, width: int, name: str = "row", window: int = 0) -> "PagedSpec":
        """One row of ``width`` elements per token."""
        return cls((PagedBuffer(name, 1, int(width)),), int(window))

    def elems_per_token(self) -> int:
        return sum(b.rows * b.width for b in self.buffers)

    def uniform(self) -> bool:
        """Whether all buffers have one shape (so that they can be read as one stacked tensor)."""
        return len({(b.rows, b.width) for b in self.buffers}) == 1


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size (``shape`` elements per layer), kept in a slot.

    ``kind`` only serves to keep unlike states in separate tensors; ``dtype`` None means the
    compute dtype.  The state of a fresh request is *undefined memory*: a mixer must derive
    "nothing before position 0" from the positions it is given, never from zeroed memory.
    """

    kind: str
    shape: Tuple[int, ...]
    dtype: Optional[torch.dtype] = None


@dataclass
class CacheView:
    """What a mixer sees of the cache at one call site of one step.

    ``paged``: ``tensor`` is this call site's pages, flat: [pages, page_size * elements per token];
    ``buffers`` names a view ``[pages, rows, page_size, width]`` of it for each
    :class:`PagedBuffer` of the mixer's spec, and :meth:`stacked` gives buffers of equal shape as
    one ``[pages, n_buffers, rows, page_size, width]`` (keys and values:
    ``[pages, 2, n_kv, page_size, head_dim]``); ``group`` has the step's ``slot_mapping`` [n]
    (page * page_size + offset of each new token) and ``block_table`` [S, width] for the layer's
    group.  ``state``: ``tensor`` is this call site's view [slots, *shape]; ``ctx.state_slots``
    [S] names each sequence's slot.  ``write`` False: the call site reads a cache another layer
    owns.
    """

    kind: str                 # "paged" | "state" | "none"
    tensor: Optional[torch.Tensor] = None
    group: Any = None
    write: bool = True
    buffers: Optional[Dict[str, torch.Tensor]] = None
    spec: Any = None

    def stacked(self) -> torch.Tensor:
        """Buffers of one shape as a single tensor [pages, n_buffers, rows, page_size, width]."""
        if self.kind == "paged" and self.tensor is not None and self.tensor.dim() == 5:
            return self.tensor               # handed over in that shape already
        if self.kind != "paged" or self.spec is None or not self.spec.uniform():
            raise ValueError("only paged buffers of equal shape can be read as one stacked tensor")
        b = self.spec.buffers[0]
        pages = self.tensor.shape[0]
        page_size = self.tensor.shape[1] // self.spec.elems_per_token()
        return self.tensor.view(pages, len(self.spec.buffers), b.rows, page_size, b.width)


@dataclass
class StreamState:
    """What the last writer of the float32 residual stream ``x`` [n, H] left for the norm that
    reads it next, in steps of a few rows (decode): ``xw`` [n, H] = bfloat16(x * that norm's
    weight) and ``ss`` [parts, n], partial sums of squares of the rows of ``x``."""

    xw: torch.Tensor
    ss: torch.Tensor


@dataclass
class NormedStream:
    """The residual stream seen through a norm that has not been applied yet.

    Decode steps are a handful of rows, so a norm of its own costs a launch for almost no
    work.  RMSNorm is ``x * w * rsqrt(mean x^2 + eps)`` and the last factor is one number per
    row, so a consumer's first matrix product can run on ``xw`` = bfloat16(x * w) and scale each
    row of its result by that number, which it gets from ``ss`` and ``eps``."""

    xw: torch.Tensor
    ss: torch.Tensor
    eps: float


# --------------------------------------------------------------------------------------
# the parts


class Part:
    """Base of every part: tensor specs and binding."""

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], prefix: str, dtype: torch.dtype) -> None:
        """Take the loaded tensors (by full checkpoint name); fuse or reshape them once."""


class Norm(Part):
    """A norm over the last dimension that also folds in the pending residual add."""

    def apply(self, x: torch.Tensor, delta: Optional[torch.Tensor], dtype: torch.dtype,
              rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x`` is the float32 residual stream [n, H].  Adds ``delta`` (a layer's output in
        the activation dtype) into it when given, and returns the normed rows in ``dtype``.
        With ``rows`` only those rows are produced and ``x`` is left unchanged."""
        raise NotImplementedError

    def stream_weight(self) -> Optional[torch.Tensor]:
        """The float32 weight vector a producer should multiply the stream by on this norm's
        behalf (see :class:`StreamState`), or None if this norm cannot be deferred."""
        return None

    def deferred(self, state: "StreamState") -> Optional[NormedStream]:
        """This norm as a :class:`NormedStream` for a consumer that applies it itself; ``state``
        must have been produced with this norm's :meth:`stream_weight`."""
        return None


class PositionEncoding(Part):
    """Prepares, once per step, what mixers need to place tokens (e.g. cos/sin rows)."""

    name: str = "pos"

    def prepare(self, ctx: "Any") -> Any:
        raise NotImplementedError


class Mixer(Part):
    """Moves information between the tokens of a sequence."""

    def cache_spec(self) -> Optional[object]:
        """A :class:`PagedSpec`, a :class:`StateSpec` or None."""
        return None

    def forward(self, a: torch.Tensor, ctx: "Any", cache: CacheView) -> torch.Tensor:
        """``a`` [n, H] normed activations of every token of the step; returns the layer's
        contribution to the residual stream, [n, H] in the activation dtype."""
        raise NotImplementedError

    def decode_splits(self, batch: int, max_context: int, page_size: int, dtype: torch.dtype) -> int:
        """Into how many slices this mixer wants a sequence's cached tokens cut in a decode step of
        ``batch`` single-token sequences whose contexts may reach ``max_context``.  Asked once per
        fixed-shape (captured) decode step, whose kernels cannot follow the batch's real lengths;
        the answer comes back to the mixer as ``cache.group.splits``.  1: no cutting."""
        return 1

    def forward_stream(self, a: NormedStream, ctx: "Any", cache: CacheView, x: torch.Tensor,
                       next_weight: torch.Tensor):
        """Optional fast form for steps of a few rows: take the normed input lazily, add the
        result into the stream ``x`` in place, and return the :class:`StreamState` of the new
        ``x`` for the norm whose weight is ``next_weight``.  Return ``NotImplemented`` to be run
        the ordinary way."""
        return NotImplemented


class FeedForward(Part):
    def forward(self, f: torch.Tensor, ctx: "Any") -> torch.Tensor:
        raise NotImplementedError

    def forward_stream(self, f: NormedStream, ctx: "Any", x: torch.Tensor, next_weight: torch.Tensor):
        """As :meth:`Mixer.forward_stream`."""
        return NotImplemented


# --------------------------------------------------------------------------------------
# registries: name -> constructor.  A new kind of part is one register_* call.

MIXERS: Dict[str, Callable[..., Mixer]] = {}
FEED_FORWARDS: Dict[str, Callable[..., FeedForward]] = {}
NORMS: Dict[str, Callable[..., Norm]] = {}
POSITION_ENCODINGS: Dict[str, Callable[..., PositionEncoding]] = {}


def _register(table: Dict[str, Callable], name: str, ctor: Callable, replace: bool) -> None:
    if name in table and not replace and table[name] is not ctor:
        raise ValueError(f"part `{name}` is already registered")
    table[name] = ctor


def register_mixer(name: str, ctor: Callable[..., Mixer], *, replace: bool = False) -> None:
    _register(MIXERS, name, ctor, replace)


def register_feed_forward(name: str, ctor: Callable[..., FeedForward], *, replace: bool = False) -> None:
    _register(FEED_FORWARDS, name, ctor, replace)


def register_norm(name: str, ctor: Callable[..., Norm], *, replace: bool = False) -> None:
    _register(NORMS, name, ctor, replace)


def register_position_encoding(name: str, ctor: Callable[..., PositionEncoding], *, replace: bool = False) -> None:
    _register(POSITION_ENCODINGS, name, ctor, replace)


def make_part(table: Dict[str, Callable], kind: str, **params: Any) -> Any:
    try:
        ctor = table[kind]
    except KeyError:
        raise KeyError(f"no part named `{kind}`; registered: {sorted(table)}")
    return ctor(**params)
