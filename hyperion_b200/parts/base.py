"""Interfaces and registries of the parts a layer is put together from.

Five kinds of part exist: mixer (attention here), feed-forward, norm, position encoding and the
arrangement of a block; embedding and output head are parts too.  A part is built from its
:class:`PartSpec` (sizes and constants only), declares the tensors it wants by name and shape,
receives them once, and then runs on the tokens of a step.  A part never learns which model it is
in.  New kinds are added with the ``register_*`` functions; nothing else has to change.

What a part must offer:

``weights() -> dict[name, WeightSpec]``   tensor names relative to its prefix, with shapes
``load(tensors)``                         the tensors, on the device, in their stored element type
``forward(...)``                          see each base class

A mixer additionally states what it keeps between steps (``cache_request``): a payload of fixed
shape per token, kept in pages (:class:`PagedTokens`; keys and values are the case :func:`PagedKV`), a
record of fixed size per request (:class:`RequestState`), or nothing.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable, Mapping, Optional

import torch

from .spec import PartSpec


@dataclass(frozen=True)
class WeightSpec:
    shape: tuple[int, ...]
    integer: bool = False  # integer tables are kept as int32, everything else as a float type
    init: str = "normal"  # how random weights fill it: "normal" = N(0, std), "one_plus_normal" = 1 + N(0, std)


@dataclass(frozen=True)
class PagedTokens:
    """A payload of fixed shape per token, kept in pages.  The cache manager gives the mixer a tensor
    [pages, *outer, page_size, *inner]: a token at position p of a request lies at
    ``[block_table[row, p // page_size], ..., p % page_size, ...]``.  ``window`` > 0: only the last
    ``window`` positions are ever read again, so older pages are given back while the request lives.
    ``dtype`` None: the model's activation type.  Users with equal requests share one pool of pages
    and one block table per request."""

    outer: tuple[int, ...] = ()
    inner: tuple[int, ...] = ()
    window: int = 0
    dtype: Optional[torch.dtype] = None

    @property
    def values_per_token(self) -> int:
        return math.prod(self.outer) * math.prod(self.inner)

    def bytes_per_token(self, activation_dtype: torch.dtype) -> int:
        return self.values_per_token * torch.empty((), dtype=self.dtype or activation_dtype).element_size()

    def storage_shape(self, num_pages: int, page_size: int) -> tuple[int, ...]:
        return (num_pages, *self.outer, page_size, *self.inner)


def PagedKV(kv_heads: int, head_dim: int, window: int = 0) -> PagedTokens:
    """Keys and values per token: pages of [2, kv_heads, page_size, head_dim]."""
    return PagedTokens((2, int(kv_heads)), (int(head_dim),), int(window))


@dataclass(frozen=True)
class RequestState:
    """A record of fixed shape per live request, zeroed when a request takes the slot."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class BuildContext:
    """What a part may know when it is built: the element type of activations and the device."""

    dtype: torch.dtype
    device: torch.device
    max_positions: int
    shared: dict  # parts may keep tables here that other parts with the same parameters reuse


class Part:
    def __init__(self, spec: PartSpec, build: BuildContext):
        self.spec = spec
        self.dtype = build.dtype
        self.device = build.device

    def weights(self) -> dict[str, WeightSpec]:
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        pass

    def kernel_modules(self) -> list[tuple[str, dict]]:
        """The native modules (name, definitions) this part launches; built before the first step."""
        return []


class Norm(Part):
    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Add ``delta`` into the float residual stream ``h`` (in place, unless ``rows`` selects rows
        to gather) and return the normalised rows in the activation type.  ``delta`` is what a mixer
        or feed-forward returned: a tensor, or a product still in its split-K pieces
        (``ops.gemm.SplitSum``; ``.tensor()`` adds them up for a norm that cannot read them itself)."""
        raise NotImplementedError


class PositionEncoding(Part):
    def apply_(self, x: torch.Tensor, heads: int, head_dim: int, positions: torch.Tensor) -> None:
        """Encode the positions into the first ``heads`` heads of every row of ``x``, in place."""
        raise NotImplementedError

    def apply_and_store_(self, x: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, positions: torch.Tensor, cache: Any,
                         token_row: torch.Tensor) -> None:
        """``x`` = [q | k | v] per token: encode q (in place) and k, and write k and v to the paged
        ``cache``.  A position encoding may fuse the three; this default does them one after the other."""
        from .. import ops

        self.apply_(x, q_heads + kv_heads, head_dim, positions)
        width = kv_heads * head_dim
        ops.kv_store(x, q_heads * head_dim, q_heads * head_dim + width, cache.kv, cache.block_table, token_row, positions)


class Mixer(Part):
    def cache_request(self) -> PagedTokens | RequestState | None:
        return None

    def forward(self, x: torch.Tensor, step: Any, cache: Any, own_cache: bool) -> torch.Tensor:
        """``x`` [tokens, hidden] in the activation type; ``step`` the step's batch description
        (:class:`hyperion_b200.engine.batch.StepContext`); ``cache`` the view of this run's cache
        (``None`` if it asked for none); ``own_cache`` false when the cache belongs to another
        schedule entry and must only be read.  Returns [tokens, hidden]."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, step: Any) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        """int32 ids -> float residual stream [tokens, hidden]."""
        raise NotImplementedError

    def shared_table(self) -> Optional[torch.Tensor]:
        """The [vocab, hidden] table a tied output head may use as its matrix, or None if this embedding has none to share."""
        return None


class Head(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Normalised rows -> float logits [rows, vocab]."""
        raise NotImplementedError

    def wants_shared_table(self) -> bool:
        """True when the head owns no matrix and takes the embedding's (``use_shared_table`` is then called after loading)."""
        return False

    def use_shared_table(self, table: torch.Tensor) -> None:
        raise NotImplementedError


class Arrangement:
    """How one layer wires its parts.  ``forward`` gets the residual stream ``h`` and a pending
    ``delta`` not yet added to it (so the add fuses with the next norm) and returns the new pair."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Mapping[str, Norm]):
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, dict(norms)

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], step: Any, cache: Any, own_cache: bool):
        raise NotImplementedError


MIXERS: dict[str, Callable[[PartSpec, BuildContext], Mixer]] = {}
FEED_FORWARDS: dict[str, Callable[[PartSpec, BuildContext], FeedForward]] = {}
NORMS: dict[str, Callable[[PartSpec, BuildContext], Norm]] = {}
POSITIONS: dict[str, Callable[[PartSpec, BuildContext], PositionEncoding]] = {}
EMBEDDINGS: dict[str, Callable[[PartSpec, BuildContext], Embedding]] = {}
HEADS: dict[str, Callable[[PartSpec, BuildContext], Head]] = {}
ARRANGEMENTS: dict[str, Callable[..., Arrangement]] = {}


def _register(table: dict, kind: str, factory: Callable) -> None:
    if kind in table and table[kind] is not factory:
        raise ValueError(f"part kind {kind!r} is already registered")
    table[kind] = factory


def register_mixer(kind: str, factory) -> None: _register(MIXERS, kind, factory)
def register_feed_forward(kind: str, factory) -> None: _register(FEED_FORWARDS, kind, factory)
def register_norm(kind: str, factory) -> None: _register(NORMS, kind, factory)
def register_position(kind: str, factory) -> None: _register(POSITIONS, kind, factory)
def register_embedding(kind: str, factory) -> None: _register(EMBEDDINGS, kind, factory)
def register_head(kind: str, factory) -> None: _register(HEADS, kind, factory)
def register_arrangement(kind: str, factory) -> None: _register(ARRANGEMENTS, kind, factory)


def make(table: dict, spec: PartSpec, build: BuildContext):
    if spec.kind not in table:
        raise KeyError(f"no part of kind {spec.kind!r} is registered (known: {sorted(table)})")
    return table[spec.kind](spec, build)
