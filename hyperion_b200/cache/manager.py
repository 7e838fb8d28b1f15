"""The cache manager: pages of keys and values with a block table per request, in groups, and
slots of fixed-size state per request.

The reference keeps one pool of pages that span all layers, a FIFO free list, a table per sequence,
growth by one page when decoding crosses a page boundary, and release of everything the moment a
sequence ends (helios/crates/helios-core/src/kv/manager.rs:99-118,183-233,324-369); next to it a
slot index per live sequence addresses fixed-size device records that are cleared on reuse
(helios/crates/helios-hal/src/backends/hopper_sm90/session.rs:191-204,581-593).  This manager keeps
those operations and adds two things the reference's single kind of layer never needed:

* *groups*: cache users with the same needs (the shape and type of what they keep per token, the
  window) share one pool of pages and one table per request; users with other needs get a pool of
  their own.  One page id addresses the same page in every member of its group.  What a user keeps
  per token is its own business: keys and values of some heads, one latent vector, anything of a
  fixed shape (:class:`hyperion_b200.parts.base.PagedTokens`).
* *windows*: a group whose users only ever read the last ``window`` positions gives a page back as
  soon as every position in it has fallen out of the window, while the request lives.

It is host code with no device dependency except the tensors it allocates when given a device; all
bookkeeping can be exercised without one.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Hashable, Optional, Sequence

import numpy as np
import torch

from .. import host
from ..host import CacheError, OutOfPages
from ..parts.base import PagedTokens, RequestState

NO_PAGE = -1


class PagePool:
    """Free list of page ids with first-in first-out reuse and double-use detection (``hb::PagePool``)."""

    def __init__(self, num_pages: int):
        self._lib = host.library()
        self._handle = ctypes.c_void_p()
        host.check(self._lib.hb_pool_new(num_pages, ctypes.byref(self._handle)))
        self.num_pages = num_pages

    def __del__(self):
        if getattr(self, "_handle", None):
            self._lib.hb_pool_delete(self._handle)
            self._handle = None

    @property
    def available(self) -> int:
        return self._lib.hb_pool_available(self._handle)

    def take(self) -> int:
        page = ctypes.c_int()
        host.check(self._lib.hb_pool_take(self._handle, ctypes.byref(page)))
        return page.value

    def give_back(self, page: int) -> None:
        host.check(self._lib.hb_pool_give_back(self._handle, page))

    def check(self) -> None:
        """Every page is either free or held, exactly once."""
        host.check(self._lib.hb_pool_check(self._handle))


@dataclass
class PagedGroup:
    spec: PagedTokens
    users: list[int]  # schedule entries whose mixers own a cache in this group, in order
    storage: Optional[torch.Tensor] = None  # [users, pages, *outer, page_size, *inner]


@dataclass
class StateGroup:
    spec: RequestState
    users: list[int]
    storage: Optional[torch.Tensor] = None  # [users, slots, *shape]


class CacheManager:
    """Groups cache users by need, owns the tensors, and keeps pages, tables, slots and lengths in
    the host runtime's ``hb::CacheIndex`` (``csrc/host/cache_index.cpp``)."""

    def __init__(self, users: Sequence[tuple[int, PagedTokens | RequestState]], page_size: int, num_pages: int, max_requests: int,
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
            if isinstance(need, PagedTokens):
                group = next((i for i, g in enumerate(self.paged) if g.spec == need), None)
                if group is None:
                    self.paged.append(PagedGroup(need, []))
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
        self.device = device
        self.dtype = dtype
        if device is not None and device.type == "cuda":
            # the reference checks --max-seq-len against the device's memory before it commits the pool
            # (helios/crates/helios-hal/src/pool_plan.rs:43-60); here the pool is refused with the numbers when it cannot fit
            wanted = num_pages * page_size * self.bytes_per_token()
            free = torch.cuda.mem_get_info(device)[0]
            if wanted > free:
                raise MemoryError(f"a cache of {num_pages * page_size} tokens needs {wanted / 2**30:.1f} GiB ({self.bytes_per_token()} bytes per token), "
                                  f"{free / 2**30:.1f} GiB are free on {device} beside the weights: lower max_tokens "
                                  f"(the command line's --max-seq-len, --max-batch or --cache-tokens)")
        if not 0 < num_pages < 2**31:
            raise ValueError(f"the number of pages must be in 1..2^31 - 1, got {num_pages}")
        self._lib = host.library()
        self._handle = ctypes.c_void_p()
        windows = host.ints([g.spec.window for g in self.paged])
        host.check(self._lib.hb_cache_new(page_size, num_pages, max_requests, len(self.paged), host.address(windows), ctypes.byref(self._handle)))
        self.keys = host.KeyMap()
        if device is not None:
            for g in self.paged:
                g.storage = torch.zeros((len(g.users), *g.spec.storage_shape(num_pages, page_size)), dtype=g.spec.dtype or dtype, device=device)
            for s in self.states:
                s.storage = torch.zeros((len(s.users), max_requests, *s.spec.shape), dtype=s.spec.dtype, device=device)

    def __del__(self):
        if getattr(self, "_handle", None):
            self._lib.hb_cache_delete(self._handle)
            self._handle = None

    @property
    def native(self) -> ctypes.c_void_p:
        """The ``HbCache*`` for calls that take the index itself (the step assembler)."""
        return self._handle

    # ------------------------------------------------------------------ lookups
    def has_user(self, entry: int) -> bool:
        """Whether the schedule entry asked for a cache of its own."""
        return entry in self._where

    def where(self, entry: int) -> tuple[str, int, int]:
        """(``"paged"`` | ``"state"``, the group, the entry's index in it)."""
        return self._where[entry]

    @property
    def group_windows(self) -> list[int]:
        """Per paged group its window (0 = it keeps every key): what the scheduler reserves pages by."""
        return [g.spec.window for g in self.paged]

    def _key(self, request: Hashable) -> int:
        key = self.keys.known(request)
        if key is None or not self._lib.hb_cache_has(self._handle, key):
            raise CacheError(f"unknown request {request!r}")
        return key

    def has(self, request: Hashable) -> bool:
        key = self.keys.known(request)
        return key is not None and bool(self._lib.hb_cache_has(self._handle, key))

    def length(self, request: Hashable) -> int:
        value = ctypes.c_int()
        host.check(self._lib.hb_cache_length(self._handle, self._key(request), ctypes.byref(value)))
        return value.value

    def slot(self, request: Hashable) -> int:
        value = ctypes.c_int()
        host.check(self._lib.hb_cache_slot(self._handle, self._key(request), ctypes.byref(value)))
        return value.value

    def table(self, group: int, request: Hashable) -> list[int]:
        """A copy of the request's block table in ``group`` (``NO_PAGE`` where a window has passed)."""
        key, size = self._key(request), ctypes.c_int()
        host.check(self._lib.hb_cache_table_size(self._handle, group, key, ctypes.byref(size)))
        pages = np.empty(size.value, dtype=np.int32)
        host.check(self._lib.hb_cache_table(self._handle, group, key, host.address(pages), size.value))
        return pages.tolist()

    @property
    def live_requests(self) -> list[Hashable]:
        keys, count = np.empty(self.max_requests, dtype=np.int64), ctypes.c_int()
        host.check(self._lib.hb_cache_live(self._handle, host.address(keys), self.max_requests, ctypes.byref(count)))
        return [self.keys.name(int(k)) for k in keys[: count.value]]

    def free_pages(self, group: int = 0) -> int:
        if not self.paged:
            return 0
        value = ctypes.c_int()
        host.check(self._lib.hb_cache_free_pages(self._handle, group, ctypes.byref(value)))
        return value.value

    def bytes_per_token(self) -> int:
        """Bytes a token costs over all paged groups and their users."""
        return sum(len(g.users) * g.spec.bytes_per_token(self.dtype) for g in self.paged)

    # ------------------------------------------------------------------ requests
    def add_request(self, request: Hashable) -> int:
        if self.has(request):
            raise CacheError(f"request {request!r} is already live")
        slot = ctypes.c_int()
        host.check(self._lib.hb_cache_add(self._handle, self.keys.key(request), ctypes.byref(slot)))
        for s in self.states:
            if s.storage is not None:
                s.storage[:, slot.value].zero_()
        return slot.value

    def pages_needed(self, request: Hashable, new_tokens: int) -> list[int]:
        """Pages each paged group must add so positions up to length + new_tokens - 1 have one."""
        need = np.zeros(max(1, len(self.paged)), dtype=np.int32)
        host.check(self._lib.hb_cache_pages_needed(self._handle, self._key(request), new_tokens, host.address(need)))
        return need[: len(self.paged)].tolist()

    def extend(self, request: Hashable, new_tokens: int) -> None:
        """Give every position of the next ``new_tokens`` tokens a page in every group, or take nothing."""
        self.extend_all([(request, new_tokens)])

    def extend_all(self, work: Sequence[tuple[Hashable, int]]) -> None:
        """``extend`` for several requests at once: all of them or none."""
        keys = host.ints([self._key(request) for request, _ in work], np.int64)
        counts = host.ints([n for _, n in work])
        self.extend_keys(keys, counts)

    def extend_keys(self, keys: np.ndarray, counts: np.ndarray) -> None:
        """``extend_all`` by runtime keys (int64) and token counts (int32)."""
        host.check(self._lib.hb_cache_extend_all(self._handle, len(keys), host.address(keys), host.address(counts)))

    def advance(self, request: Hashable, new_tokens: int) -> list[tuple[int, int]]:
        """The tokens are written: move the length and give back pages a window has passed.
        Returns the (group, page) pairs released."""
        key, count = self._key(request), ctypes.c_int()
        length = self.length(request)
        capacity = (length + new_tokens) // self.page_size * max(1, len(self.paged)) + 1  # no more blocks than that exist
        pairs = np.empty(2 * capacity, dtype=np.int32)
        host.check(self._lib.hb_cache_advance(self._handle, key, new_tokens, host.address(pairs), capacity, ctypes.byref(count)))
        return [(int(pairs[2 * i]), int(pairs[2 * i + 1])) for i in range(count.value)]

    def advance_keys(self, keys: np.ndarray, counts: np.ndarray) -> None:
        host.check(self._lib.hb_cache_advance_all(self._handle, len(keys), host.address(keys), host.address(counts)))

    def free(self, request: Hashable) -> None:
        key = self.keys.known(request)
        if key is None or not self._lib.hb_cache_has(self._handle, key):
            raise CacheError(f"request {request!r} is not live")
        host.check(self._lib.hb_cache_free(self._handle, key))
        self.keys.forget(request)

    def check(self) -> None:
        """Accounting invariants: no page lost or held twice; every held page is in exactly one table."""
        host.check(self._lib.hb_cache_check(self._handle))

    # ------------------------------------------------------------------ views for the parts
    def paged_storage(self, entry: int) -> torch.Tensor:
        kind, group, index = self._where[entry]
        assert kind == "paged"
        return self.paged[group].storage[index]

    def state_storage(self, entry: int) -> torch.Tensor:
        kind, group, index = self._where[entry]
        assert kind == "state"
        return self.states[group].storage[index]
