"""The cache manager: pages of keys and values with a block table per request, in groups, and
slots of fixed-size state per request.

The reference keeps one pool of pages that span all layers, a FIFO free list, a table per sequence,
growth by one page when decoding crosses a page boundary, and release of everything the moment a
sequence ends (helios/crates/helios-core/src/kv/manager.rs:99-118,183-233,324-369); next to it a
slot index per live sequence addresses fixed-size device records that are cleared on reuse
(helios/crates/helios-hal/src/backends/hopper_sm90/session.rs:191-204,581-593).  This manager keeps
those operations and adds two things the reference's single kind of layer never needed:

* *groups*: cache users with the same needs (key/value heads, head size, window) share one pool of
  pages and one table per request; users with other needs get a pool of their own.  One page id
  addresses the same page in every member of its group.
* *windows*: a group whose users only ever read the last ``window`` positions gives a page back as
  soon as every position in it has fallen out of the window, while the request lives.

It is host code with no device dependency except the tensors it allocates when given a device; all
bookkeeping can be exercised without one.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Hashable, Optional, Sequence

import torch

from ..parts.base import PagedKV, RequestState

NO_PAGE = -1


class OutOfPages(RuntimeError):
    """A request asked for more pages than its group's pool has free; nothing was taken."""


class CacheError(RuntimeError):
    """The manager was used inconsistently (unknown request, page freed twice, ...)."""


class PagePool:
    """Free list of page ids with first-in first-out reuse and double-use detection."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: deque[int] = deque(range(num_pages))
        self._held: set[int] = set()

    @property
    def available(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.popleft()
        self._held.add(page)
        return page

    def give_back(self, page: int) -> None:
        if page not in self._held:
            raise CacheError(f"page {page} given back but not held")
        self._held.remove(page)
        self._free.append(page)

    def check(self) -> None:
        """Every page is either free or held, exactly once."""
        free = list(self._free)
        if len(set(free)) != len(free) or set(free) & self._held or len(free) + len(self._held) != self.num_pages:
            raise CacheError("page accounting broken")


@dataclass
class PagedGroup:
    spec: PagedKV
    users: list[int]  # schedule entries whose mixers own a cache in this group, in order
    pool: PagePool
    tables: dict[Hashable, list[int]] = field(default_factory=dict)
    storage: Optional[torch.Tensor] = None  # [users, pages, 2, kv_heads, page_size, head_dim]


@dataclass
class StateGroup:
    spec: RequestState
    users: list[int]
    storage: Optional[torch.Tensor] = None  # [users, slots, *shape]


@dataclass
class _Request:
    slot: int
    length: int = 0  # tokens whose cache entries are written


class CacheManager:
    def __init__(self, users: Sequence[tuple[int, PagedKV | RequestState]], page_size: int, num_pages: int, max_requests: int,
                 dtype: torch.dtype = torch.float32, device: Optional[torch.device] = None):
        if page_size <= 0 or page_size & (page_size - 1):
            raise ValueError(f"page_size must be a power of two, got {page_size}")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.paged: list[PagedGroup] = []
        self.states: list[StateGroup] = []
        self._where: dict[int, tuple[str, int, int]] = {}  # schedule entry -> (kind, group, index in group)
        for entry, need in users:
            if isinstance(need, PagedKV):
                group = next((i for i, g in enumerate(self.paged) if g.spec == need), None)
                if group is None:
                    self.paged.append(PagedGroup(need, [], PagePool(num_pages)))
                    group = len(self.paged) - 1
                self.paged[group].users.append(entry)
                self._where[entry] = ("paged", group, len(self.paged[group].users) - 1)
            elif isinstance(need, RequestState):
                group = next((i for i, g in enumerate(self.states) if g.spec == need), None)
                if group is None:
                    self.states.append(StateGroup(need, []))
                    group = len(self.states) - 1
                self.states[group].users.append(entry)
                self._where[entry] = ("state", group, len(self.states[group].users) - 1)
            else:
                raise TypeError(f"unknown cache request {need!r}")
        self._requests: dict[Hashable, _Request] = {}
        self._free_slots: deque[int] = deque(range(max_requests))
        self.device = device
        if device is not None:
            for g in self.paged:
                g.storage = torch.zeros((len(g.users), num_pages, 2, g.spec.kv_heads, page_size, g.spec.head_dim), dtype=dtype, device=device)
            for s in self.states:
                s.storage = torch.zeros((len(s.users), max_requests, *s.spec.shape), dtype=s.spec.dtype, device=device)

    # ------------------------------------------------------------------ lookups
    def where(self, entry: int) -> tuple[str, int, int]:
        return self._where[entry]

    def has(self, request: Hashable) -> bool:
        return request in self._requests

    def length(self, request: Hashable) -> int:
        return self._requests[request].length

    def slot(self, request: Hashable) -> int:
        return self._requests[request].slot

    def table(self, group: int, request: Hashable) -> list[int]:
        return self.paged[group].tables[request]

    @property
    def live_requests(self) -> list[Hashable]:
        return list(self._requests)

    def free_pages(self, group: int = 0) -> int:
        return self.paged[group].pool.available if self.paged else 0

    def bytes_per_token(self) -> int:
        total = 0
        for g in self.paged:
            itemsize = g.storage.element_size() if g.storage is not None else 2
            total += len(g.users) * 2 * g.spec.kv_heads * g.spec.head_dim * itemsize
        return total

    # ------------------------------------------------------------------ requests
    def add_request(self, request: Hashable) -> int:
        if request in self._requests:
            raise CacheError(f"request {request!r} is already live")
        if not self._free_slots:
            raise OutOfPages(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.popleft()
        self._requests[request] = _Request(slot)
        for g in self.paged:
            g.tables[request] = []
        for s in self.states:
            if s.storage is not None:
                s.storage[:, slot].zero_()
        return slot

    def _first_needed_block(self, group: PagedGroup, length: int) -> int:
        """The first block a query at position ``length`` (the next one) can still read."""
        if group.spec.window <= 0:
            return 0
        return max(0, length - group.spec.window + 1) // self.page_size

    def pages_needed(self, request: Hashable, new_tokens: int) -> list[int]:
        """Pages each paged group must add so positions up to length + new_tokens - 1 have one."""
        length = self._requests[request].length
        blocks = -(-(length + new_tokens) // self.page_size)
        return [max(0, blocks - len(g.tables[request])) for g in self.paged]

    def extend(self, request: Hashable, new_tokens: int) -> None:
        """Give every position of the next ``new_tokens`` tokens a page in every group, or take nothing."""
        need = self.pages_needed(request, new_tokens)
        for g, n in zip(self.paged, need):
            if n > g.pool.available:
                raise OutOfPages(f"request {request!r} needs {n} more pages, {g.pool.available} free")
        for g, n in zip(self.paged, need):
            g.tables[request].extend(g.pool.take() for _ in range(n))

    def extend_all(self, work: Sequence[tuple[Hashable, int]]) -> None:
        """``extend`` for several requests at once: all of them or none."""
        totals = [0] * len(self.paged)
        for request, n in work:
            if request not in self._requests:
                raise CacheError(f"unknown request {request!r}")
            for i, pages in enumerate(self.pages_needed(request, n)):
                totals[i] += pages
        for g, n in zip(self.paged, totals):
            if n > g.pool.available:
                raise OutOfPages(f"the step needs {n} more pages, {g.pool.available} free")
        for request, n in work:
            self.extend(request, n)

    def advance(self, request: Hashable, new_tokens: int) -> list[tuple[int, int]]:
        """The tokens are written: move the length and give back pages a window has passed.
        Returns the (group, page) pairs released."""
        record = self._requests[request]
        record.length += new_tokens
        released = []
        for index, g in enumerate(self.paged):
            table = g.tables[request]
            if len(table) * self.page_size < record.length:
                raise CacheError(f"request {request!r} advanced past its pages")
            for block in range(min(self._first_needed_block(g, record.length), len(table))):
                if table[block] != NO_PAGE:
                    g.pool.give_back(table[block])
                    released.append((index, table[block]))
                    table[block] = NO_PAGE
        return released

    def free(self, request: Hashable) -> None:
        record = self._requests.pop(request, None)
        if record is None:
            raise CacheError(f"request {request!r} is not live")
        for g in self.paged:
            for page in g.tables.pop(request):
                if page != NO_PAGE:
                    g.pool.give_back(page)
        self._free_slots.append(record.slot)

    def check(self) -> None:
        """Accounting invariants: no page lost or held twice; every held page is in exactly one table."""
        for g in self.paged:
            g.pool.check()
            seen: set[int] = set()
            for table in g.tables.values():
                for page in table:
                    if page == NO_PAGE:
                        continue
                    if page in seen:
                        raise CacheError(f"page {page} is in two tables")
                    seen.add(page)
            if seen != g.pool._held:
                raise CacheError("held pages and tables disagree")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots) or len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("slot accounting broken")

    # ------------------------------------------------------------------ views for the parts
    def paged_storage(self, entry: int) -> torch.Tensor:
        kind, group, index = self._where[entry]
        assert kind == "paged"
        return self.paged[group].storage[index]

    def state_storage(self, entry: int) -> torch.Tensor:
        kind, group, index = self._where[entry]
        assert kind == "state"
        return self.states[group].storage[index]
