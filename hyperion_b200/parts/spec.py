"""A model as data: which parts each layer is made of, with their sizes and constants, and the
order in which layers run.

An architecture turns its typed configuration into a :class:`ModelSpec`; nothing below this file
knows which architecture it serves.  The reference builds one fixed stack of identical layers in
code (helios/crates/helios-hal/src/backends/hopper_sm90/session.rs:646-811); here the stack is a
list, so a model may mix kinds of mixer and feed-forward, run a layer twice, or let a layer read
the cache another layer wrote.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered ``kind``, the prefix of its tensor names, and its parameters."""

    kind: str
    prefix: str = ""
    params: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (how norms, mixer and feed-forward are wired) and its parts."""

    arrangement: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Mapping[str, PartSpec]


@dataclass(frozen=True)
class Run:
    """One entry of the schedule: run ``layer``; its mixer owns a cache of its own unless
    ``reads_cache_of`` names an earlier schedule entry whose cache it reads instead."""

    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[Run, ...]
    final_norm: PartSpec
    head: PartSpec
    # tensor names a checkpoint may carry without their being used (for instance the output matrix
    # of a checkpoint with tied embeddings)
    tolerated: tuple[str, ...] = ()

    def validate(self) -> None:
        for index, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule[{index}] names layer {run.layer}, the model has {len(self.layers)}")
            if run.reads_cache_of is not None:
                if not 0 <= run.reads_cache_of < index:
                    raise ValueError(f"schedule[{index}] must read the cache of an earlier entry, got {run.reads_cache_of}")
                if self.schedule[run.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(f"schedule[{index}] reads the cache of an entry that owns none")
