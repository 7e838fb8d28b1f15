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

import ctypes
from collections.abc import Sequence
from dataclasses import dataclass, field
from typing import Any, Hashable, Optional

import numpy as np
import torch

from .. import host as host_runtime


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


class Rows(Sequence):
    """The rows of a step as arrays (``starts``, ``counts``, ``positions``, ``slots``: int32, one entry
    per row); indexing or iterating gives :class:`Row` objects, made when asked for."""

    def __init__(self, names: Sequence[Hashable], starts: np.ndarray, counts: np.ndarray, positions: np.ndarray, slots: np.ndarray):
        self.names, self.starts, self.counts, self.positions, self.slots = names, starts, counts, positions, slots

    def __len__(self) -> int:
        return len(self.counts)

    def __getitem__(self, index):
        if isinstance(index, slice):
            return [self[i] for i in range(*index.indices(len(self)))]
        return Row(self.names[index], int(self.starts[index]), int(self.counts[index]), int(self.positions[index]), int(self.slots[index]))

    @property
    def longest_context(self) -> int:
        """The largest position any row reaches in this step, plus one."""
        return int((self.positions + self.counts).max())


@dataclass
class PagedView:
    """What a mixer with a paged cache request is handed: its own pages and the step's block tables of its group."""

    storage: torch.Tensor  # [pages, *outer, page_size, *inner] of this schedule entry (keys and values: [pages, 2, kv_heads, page_size, head_dim])
    block_table: torch.Tensor  # [rows, width] int32 on the device
    page_size: int
    group: int

    @property
    def kv(self) -> torch.Tensor:
        """The same tensor, under the name attention parts use."""
        return self.storage


@dataclass
class StateView:
    state: torch.Tensor  # [slots, *shape] of this schedule entry
    slots: torch.Tensor  # [rows] int32 on the device
    row_slots: list[int]


def _dense_strides(shape: tuple[int, ...]) -> tuple[int, ...]:
    strides, step = [], 1
    for extent in reversed(shape):
        strides.append(step)
        step *= extent
    return tuple(reversed(strides))


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
        self.generation = 0  # counts reallocations of the device buffer
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
        self._recorded = [False] * self.RING  # whether the slot's event stands for a copy that may still be reading it
        self._host_words = [host.numpy() for host in self.hosts]
        self.dev = torch.empty(capacity, dtype=torch.int32, device=self.device)
        self.generation += 1

    def begin(self) -> None:
        """Take the next staging buffer of the ring (waiting for the copy that last read it) and start an empty layout."""
        self._items: list[tuple[str, int, int, tuple[int, ...]]] = []
        self._cursor = 0
        self._index = (self._index + 1) % self.RING
        if self._recorded[self._index]:
            self.events[self._index].synchronize()
            self._recorded[self._index] = False
        self._words = self._host_words[self._index]

    def _grow(self, needed: int) -> None:
        """More room than the buffers have: new buffers (``generation`` tells users of the device buffer), what is written so far kept."""
        written = self._words[: self._cursor].copy()
        self._reserve(max(needed, 2 * self.capacity))
        self._words = self._host_words[self._index]
        self._words[: self._cursor] = written

    def add(self, name: str, values: Any, shape: Optional[tuple[int, ...]] = None) -> None:
        """Append an int32 array (a list of ints, a numpy array or a tensor); every array starts on a 16-byte boundary."""
        if isinstance(values, torch.Tensor):
            values = values.detach().cpu().numpy()
        array = np.asarray(values, dtype=np.int32).reshape(-1)
        count = array.size
        start = (self._cursor + 3) & ~3
        if start + count > self.capacity:
            self._grow(start + count)
        self._words[start : start + count] = array
        self._items.append((name, start, count, shape or (count,)))
        self._cursor = start + count

    def add_step(self, cache, keys: np.ndarray, counts: np.ndarray, tokens: np.ndarray, want: np.ndarray, table_step: int) -> None:
        """The arrays every step carries, written by the host runtime's step assembler straight into the staging
        buffer: token_ids, positions, token_row, row_start, slots, want and one block table per paged group."""
        groups = len(cache.paged)
        layout = np.zeros(4 * (6 + groups), dtype=np.int64)
        lib = host_runtime.library()
        for attempt in range(2):
            cursor = ctypes.c_int64(self._cursor)
            code = lib.hb_step_pack(cache.native, len(keys), host_runtime.address(keys), host_runtime.address(counts), host_runtime.address(tokens),
                                    len(want), host_runtime.address(want), table_step, self._words.ctypes.data, self.capacity, ctypes.byref(cursor),
                                    host_runtime.address(layout))
            if code == host_runtime.BAD_ARGUMENT and attempt == 0 and b"metadata needs" in lib.hb_host_last_error():
                self._grow(int(lib.hb_host_last_error().split()[-2]))
                continue
            host_runtime.check(code)
            break
        self._cursor = cursor.value
        names = ["token_ids", "positions", "token_row", "row_start", "slots", "want"] + [f"table{g}" for g in range(groups)]
        for index, name in enumerate(names):
            offset, count, rows, columns = (int(v) for v in layout[4 * index : 4 * index + 4])
            if name == "want" and count == 0:
                continue
            self._items.append((name, offset, count, (rows, columns) if name.startswith("table") else (count,)))

    def view(self, name: str) -> np.ndarray:
        """What was written under ``name`` in the staging buffer of this step (host side)."""
        for item, start, count, shape in self._items:
            if item == name:
                return self._words[start : start + count].reshape(shape)
        raise KeyError(name)

    def finish(self) -> dict[str, torch.Tensor]:
        if self._cursor:
            self.dev[: self._cursor].copy_(self.hosts[self._index][: self._cursor], non_blocking=True)
            if self.device.type == "cuda":
                if self.events[self._index] is None:
                    self.events[self._index] = torch.cuda.Event()
                self.events[self._index].record()
                self._recorded[self._index] = True
        dev = self.dev
        return {name: dev.as_strided(shape, _dense_strides(shape), start) for name, start, count, shape in self._items}


@dataclass
class StepContext:
    rows: Rows
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
