"""Binding of the C++ host runtime (``csrc/host``): cache index, scheduler and step assembly.

The C++ classes hold all bookkeeping; the Python classes of ``cache`` and ``engine`` are thin
faces over them that keep request names (any hashable) and tensors.  The library is compiled with
the system's C++ compiler on first use; there is no Python stand-in for it.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_char_p, c_int, c_int32, c_int64, c_void_p
from typing import Hashable

import numpy as np

from ..csrc import build


class OutOfPages(RuntimeError):
    """A request asked for more pages (or request slots) than are free; nothing was taken."""


class CacheError(RuntimeError):
    """The cache was used inconsistently (unknown request, page freed twice, ...)."""


class QueueFull(RuntimeError):
    pass


OK, OUT_OF_PAGES, CACHE_ERROR, BAD_ARGUMENT, BAD_STEP, QUEUE_FULL, SCHEDULER_ERROR, BAD_FILE = range(8)
_ERRORS = {OUT_OF_PAGES: OutOfPages, CACHE_ERROR: CacheError, BAD_ARGUMENT: ValueError, QUEUE_FULL: QueueFull, SCHEDULER_ERROR: RuntimeError}

_library = None
I32P, I64P = POINTER(c_int), POINTER(c_int64)


def library() -> ctypes.CDLL:
    global _library
    if _library is None:
        lib = build.load_host()
        lib.hb_host_last_error.restype = c_char_p
        for name in ("hb_pool_delete", "hb_cache_delete", "hb_sched_delete", "hb_safetensors_close"):
            getattr(lib, name).restype = None
            getattr(lib, name).argtypes = [c_void_p]
        lib.hb_pool_new.argtypes = [c_int, POINTER(c_void_p)]
        lib.hb_pool_available.argtypes = [c_void_p]
        lib.hb_pool_take.argtypes = [c_void_p, I32P]
        lib.hb_pool_give_back.argtypes = [c_void_p, c_int]
        lib.hb_pool_is_held.argtypes = [c_void_p, c_int]
        lib.hb_pool_check.argtypes = [c_void_p]
        lib.hb_cache_new.argtypes = [c_int, c_int, c_int, c_int, c_void_p, POINTER(c_void_p)]
        lib.hb_cache_has.argtypes = [c_void_p, c_int64]
        lib.hb_cache_add.argtypes = [c_void_p, c_int64, I32P]
        lib.hb_cache_length.argtypes = [c_void_p, c_int64, I32P]
        lib.hb_cache_slot.argtypes = [c_void_p, c_int64, I32P]
        lib.hb_cache_table_size.argtypes = [c_void_p, c_int, c_int64, I32P]
        lib.hb_cache_table.argtypes = [c_void_p, c_int, c_int64, c_void_p, c_int]
        lib.hb_cache_pages_needed.argtypes = [c_void_p, c_int64, c_int, c_void_p]
        lib.hb_cache_extend_all.argtypes = [c_void_p, c_int, c_void_p, c_void_p]
        lib.hb_cache_advance.argtypes = [c_void_p, c_int64, c_int, c_void_p, c_int, I32P]
        lib.hb_cache_advance_all.argtypes = [c_void_p, c_int, c_void_p, c_void_p]
        lib.hb_cache_free.argtypes = [c_void_p, c_int64]
        lib.hb_cache_free_pages.argtypes = [c_void_p, c_int, I32P]
        lib.hb_cache_live.argtypes = [c_void_p, c_void_p, c_int, I32P]
        lib.hb_cache_lengths.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p]
        lib.hb_cache_check.argtypes = [c_void_p]
        lib.hb_step_pack.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int64, POINTER(c_int64), c_void_p]
        lib.hb_step_decode_widths.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p]
        lib.hb_plan_attention.argtypes = [c_int, c_void_p, c_int, c_int, c_void_p, I32P, c_void_p, I32P]
        lib.hb_cache_worst_case_pages.argtypes = [c_int, c_int, c_int, c_int, I32P]
        lib.hb_sched_new.argtypes = [c_int, c_int, c_int, c_void_p] + [c_int] * 7 + [c_void_p, POINTER(c_void_p)]
        lib.hb_sched_enqueue.argtypes = [c_void_p, c_int64, c_int, c_void_p, c_int, c_int]
        lib.hb_sched_next_plan.argtypes = [c_void_p, I32P, I32P, I32P]
        lib.hb_sched_plan.argtypes = [c_void_p, c_int] + [c_void_p] * 7
        lib.hb_sched_complete.argtypes = [c_void_p, c_int, c_int, c_void_p]
        lib.hb_sched_fail.argtypes = [c_void_p, c_int, c_char_p]
        lib.hb_sched_cancel.argtypes = [c_void_p, c_int64, I32P]
        lib.hb_sched_take_events.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, I32P, I32P]
        lib.hb_sched_take_released.argtypes = [c_void_p, c_int, c_void_p, I32P]
        lib.hb_sched_state.argtypes = [c_void_p, I32P, I32P, I32P, I32P, I32P]
        lib.hb_sched_waiting_keys.argtypes = [c_void_p, c_void_p, c_int]
        lib.hb_safetensors_open.argtypes = [c_char_p, POINTER(c_void_p)]
        lib.hb_safetensors_count.argtypes = [c_void_p]
        lib.hb_safetensors_payload_start.argtypes = [c_void_p]
        lib.hb_safetensors_payload_start.restype = c_int64
        lib.hb_safetensors_entry.argtypes = [c_void_p, c_int, POINTER(c_char_p), POINTER(c_char_p), I32P, POINTER(I64P), I64P, I64P]
        _library = lib
    return _library


def check(code: int, errors: dict | None = None) -> None:
    """Raise the Python exception that stands for a non-zero code of the runtime, with its text."""
    if code == OK:
        return
    message = (library().hb_host_last_error() or b"").decode("utf-8", "replace")
    kind = (errors or {}).get(code) or _ERRORS.get(code, RuntimeError)
    raise kind(message)


def safetensors_header(path: str, error: type) -> tuple[int, list[tuple[str, str, tuple[int, ...], int, int]]]:
    """(payload start, [(name, dtype, shape, begin, end)]) of one safetensors file, read and checked by the runtime;
    a file that fails a check raises ``error`` with the runtime's text."""
    lib = library()
    table = c_void_p()
    check(lib.hb_safetensors_open(str(path).encode("utf-8"), byref(table)), {BAD_FILE: error})
    try:
        entries = []
        name, dtype, rank, shape, begin, end = c_char_p(), c_char_p(), c_int(), I64P(), c_int64(), c_int64()
        for index in range(lib.hb_safetensors_count(table)):
            check(lib.hb_safetensors_entry(table, index, byref(name), byref(dtype), byref(rank), byref(shape), byref(begin), byref(end)))
            entries.append((name.value.decode("utf-8"), dtype.value.decode("ascii"), tuple(int(shape[d]) for d in range(rank.value)),
                            int(begin.value), int(end.value)))
        return int(lib.hb_safetensors_payload_start(table)), entries
    finally:
        lib.hb_safetensors_close(table)


def ints(values, dtype=np.int32) -> np.ndarray:
    """A contiguous array of the runtime's integer type over ``values`` (no copy when it already is one)."""
    return np.ascontiguousarray(values, dtype=dtype)


def address(array: np.ndarray) -> int:
    return array.ctypes.data


class KeyMap:
    """Request names (any hashable) <-> the 64-bit keys the runtime knows them by."""

    def __init__(self):
        self._key_of: dict[Hashable, int] = {}
        self._name_of: dict[int, Hashable] = {}
        self._next = 0

    def key(self, name: Hashable) -> int:
        """The key of a name, made on first sight."""
        key = self._key_of.get(name)
        if key is None:
            key = self._next
            self._next += 1
            self._key_of[name] = key
            self._name_of[key] = name
        return key

    def known(self, name: Hashable):
        return self._key_of.get(name)

    def name(self, key: int) -> Hashable:
        return self._name_of[key]

    def forget(self, name: Hashable) -> None:
        key = self._key_of.pop(name, None)
        if key is not None:
            del self._name_of[key]
