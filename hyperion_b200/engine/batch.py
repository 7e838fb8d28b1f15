"""What one step carries: the entries (request, its next tokens, where logits are wanted) and the
flattened description of the batch that the parts read on the device.

The reference's step plan is either one prompt chunk or a bucket of single decode tokens, never
both (helios/crates/helios-hal/src/step.rs:19-60,92-99; the mixed form is only designed in
docs/decisions/0011-mixed-prefill-decode-steps.md).  Here a step is one flat batch of tokens: any
number of rows, each a request with n >= 1 next tokens starting at the position its cache has
reached.  All integer metadata of a step is packed into one pinned buffer and copied to the device
with a single transfer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Hashable, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    """``tokens`` are the request's next tokens; ``want`` the indices among them whose logits are asked for."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class BadStep(ValueError):
    """The step was refused as a whole; nothing of it was applied."""


@dataclass
class Row:
    request: Hashable
    start: int  # index of the row's first token in the flat batch
    count: int
    position: int  # position of its first token
    slot: int


@dataclass
class PagedView:
    kv: torch.Tensor  # [pages, 2, kv_heads, page_size, head_dim] of this schedule entry
    block_table: torch.Tensor  # [rows, width] int32 on the device
    page_size: int
    group: int


@dataclass
class StateView:
    state: torch.Tensor  # [slots, *shape] of this schedule entry
    slots: torch.Tensor  # [rows] int32 on the device
    row_slots: list[int]


class MetadataPacker:
    """Collects int32 arrays on the host and hands back device views after one copy.

    The pinned staging buffers form a ring: a buffer is written again only after the copy that read
    it last has completed, so the host may run several steps ahead of the device."""

    RING = 4

    def __init__(self, device: torch.device, capacity: int = 1 << 16):
        self.device = device
        self.capacity = 0
        self.hosts: list[torch.Tensor] = []
        self.events: list[Optional[torch.cuda.Event]] = [None] * self.RING
        self.dev: Optional[torch.Tensor] = None
        self._index = 0
        self._reserve(capacity)

    def _reserve(self, capacity: int) -> None:
        if capacity <= self.capacity:
            return
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        self.capacity = capacity
        self.hosts = [torch.empty(capacity, dtype=torch.int32, pin_memory=self.device.type == "cuda") for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.dev = torch.empty(capacity, dtype=torch.int32, device=self.device)

    def begin(self) -> None:
        self._items: list[tuple[str, int, int, tuple[int, ...]]] = []
        self._cursor = 0
        self._chunks: list[np.ndarray] = []

    def add(self, name: str, values: Any, shape: Optional[tuple[int, ...]] = None) -> None:
        """Append an int32 array (a list of ints, a numpy array or a tensor); every array starts on a 16-byte boundary."""
        if isinstance(values, torch.Tensor):
            values = values.detach().cpu().numpy()
        array = np.asarray(values, dtype=np.int32).reshape(-1)
        count = array.size
        shape = shape or (count,)
        self._items.append((name, self._cursor, count, shape))
        self._chunks.append(array)
        padding = -count % 4
        if padding:
            self._chunks.append(np.zeros(padding, dtype=np.int32))
        self._cursor += count + padding

    def finish(self) -> dict[str, torch.Tensor]:
        if self._cursor > self.capacity:
            self._reserve(max(self._cursor, 2 * self.capacity))
        self._index = (self._index + 1) % self.RING
        if self.events[self._index] is not None:
            self.events[self._index].synchronize()
        host = self.hosts[self._index]
        if self._cursor:
            np.concatenate(self._chunks, out=host.numpy()[: self._cursor])  # straight into the pinned buffer
            self.dev[: self._cursor].copy_(host[: self._cursor], non_blocking=True)
            if self.device.type == "cuda":
                event = torch.cuda.Event()
                event.record()
                self.events[self._index] = event
        return {name: self.dev[start : start + count].view(shape) for name, start, count, shape in self._items}


@dataclass
class StepContext:
    rows: list[Row]
    n_tokens: int
    token_ids: torch.Tensor  # [T] int32
    positions: torch.Tensor  # [T] int32
    token_row: torch.Tensor  # [T] int32: the row each token belongs to
    row_start: torch.Tensor  # [R + 1] int32
    want_rows: Optional[torch.Tensor]  # [W] int32: flat token indices whose logits are wanted
    n_want: int
    paged_tables: list[torch.Tensor]  # per paged group: [R, width] int32
    slots: torch.Tensor  # [R] int32
    extra: dict[str, torch.Tensor] = field(default_factory=dict)  # what planners of parts added
    host: dict[str, Any] = field(default_factory=dict)

    @property
    def n_rows(self) -> int:
        return len(self.rows)
