"""The scheduler's Python face: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

It is a state machine without clock, thread or device, so that the same trace of requests always
yields the same plans, like the reference's step scheduler
(helios/crates/helios-core/src/step_scheduler.rs:1-3,92-154).  Policies taken from it:

* first-in first-out queue with a bound (step_scheduler.rs:113-124);
* admission by worst-case reservation: a newcomer's pages for ``min(prompt + max_tokens,
  max_seq_len)`` tokens must fit beside what the running requests have reserved, else it waits; a
  request that could never fit is failed at once (step_scheduler.rs:160-201).  Pages therefore never
  run out under a running request, and there is no preemption, swap or recompute;
* the oldest prompt is served first, and while requests are decoding a prompt portion is at most
  ``prefill_chunk_busy`` tokens (step_scheduler.rs:206-213,238-241);
* an end-of-sequence token ends a request and is not emitted; ``max_tokens`` or the context limit
  end it with reason ``length``; pages and slot are released at once (step_scheduler.rs:364-383).

Unlike the reference, whose step is either one prompt chunk or a bucket of decode rows, a step here
mixes both: every decoding request contributes its one token, and prompt portions fill what is
left of the step's token budget, so portion sizes change from step to step.

Plans may run ahead of their results (``max_in_flight`` > 1): everything a plan needs except the
value of the token sampled by the plan before it is known when that plan was made (how many tokens
a request has, whether ``max_tokens`` or the context limit ends it).  A row whose token is still
on the device carries ``PENDING_TOKEN`` and names the plan and sampled row it comes from; the
engine feeds it from the device.  Only an end-of-sequence token is learnt late: the request then
has one row too many in flight, whose result is dropped.

The state machine itself is ``hb::Scheduler`` of the host runtime (``csrc/host/scheduler.cpp``); this
module keeps request names and sampling parameters and turns its arrays into the objects below.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Hashable, Optional, Sequence

import numpy as np

from .. import host
from ..host import QueueFull
from ..sampling.params import SamplingParams

PENDING_TOKEN = -1  # stands in a plan row for a sampled token that has not reached the host yet
EVENT_KINDS = ("token", "finished", "failed")
MAX_TOKENS_LIMIT = 2**31 - 1


@dataclass
class Request:
    id: Hashable
    prompt: Sequence[int]
    params: SamplingParams


@dataclass
class SchedulerConfig:
    num_pages: int
    page_size: int
    max_seq_len: int
    max_batch: int = 64  # most requests live at a time
    max_batch_tokens: int = 2048  # token budget of one step
    prefill_chunk_busy: int = 512  # largest prompt portion while requests are decoding
    max_queue: int = 1 << 16
    eos_token_ids: tuple[int, ...] = ()
    max_in_flight: int = 1  # plans that may be made before the oldest one's results are in
    # one entry per paged group of the cache, 0 = the group keeps every key, else its window; pages are reserved per
    # group (a windowed group costs what its window and one portion span, a model without paged groups nothing)
    group_windows: tuple[int, ...] = (0,)


@dataclass
class PlanRow:
    request: Hashable
    tokens: list[int]
    sample: bool  # the row's last token ends the prompt or is a decode token: a token is chosen after it
    sampled_before: int  # how many tokens the request has sampled so far (the draw counter)
    token_from: Optional[tuple[int, int]] = None  # tokens == [PENDING_TOKEN]: (plan step, index among its sampled rows)


@dataclass
class Plan:
    step: int
    rows: list[PlanRow]


@dataclass
class PlanArrays:
    """A plan as the runtime hands it out: one entry per row, tokens of all rows back to back."""

    step: int
    keys: np.ndarray  # int64 runtime keys of the rows' requests
    counts: np.ndarray
    sample: np.ndarray
    sampled_before: np.ndarray
    from_step: np.ndarray  # -1 unless the row's token is still on the device
    from_index: np.ndarray
    tokens: np.ndarray


@dataclass
class Event:
    request: Hashable
    kind: str  # "token" | "finished" | "failed"
    token: Optional[int] = None
    reason: Optional[str] = None  # "stop" | "length" | "cancelled" | message of a failure


class Scheduler:
    def __init__(self, config: SchedulerConfig):
        self.config = config
        self._lib = host.library()
        self._handle = ctypes.c_void_p()
        eos = host.ints(list(config.eos_token_ids))
        windows = host.ints(list(config.group_windows))
        host.check(self._lib.hb_sched_new(config.num_pages, config.page_size, len(windows), host.address(windows), config.max_seq_len, config.max_batch,
                                          config.max_batch_tokens,
                                          config.prefill_chunk_busy, config.max_queue, config.max_in_flight, len(eos), host.address(eos),
                                          ctypes.byref(self._handle)))
        self.keys = host.KeyMap()
        self.requests: dict[int, Request] = {}  # by runtime key, until the request's last event has been taken
        self._released: list[Hashable] = []

    def __del__(self):
        if getattr(self, "_handle", None):
            self._lib.hb_sched_delete(self._handle)
            self._handle = None

    # ------------------------------------------------------------------ intake
    def enqueue(self, request: Request) -> int:
        """Queue a request; returns the key the runtime knows it by."""
        if self.keys.known(request.id) is not None:
            raise ValueError(f"request id {request.id!r} is already known")
        if not 0 < request.params.max_tokens <= MAX_TOKENS_LIMIT:  # the runtime takes it as a 32-bit int
            raise ValueError(f"max_tokens must be in 1..={MAX_TOKENS_LIMIT}, got {request.params.max_tokens}")
        key = self.keys.key(request.id)
        prompt = host.ints(list(request.prompt))
        try:
            host.check(self._lib.hb_sched_enqueue(self._handle, key, len(prompt), host.address(prompt), request.params.max_tokens,
                                                  int(request.params.ignore_eos)))
        except Exception:
            self.keys.forget(request.id)
            raise
        self.requests[key] = request
        return key

    def _state(self) -> tuple[int, int, int, int, int]:
        values = [ctypes.c_int() for _ in range(5)]
        host.check(self._lib.hb_sched_state(self._handle, *[ctypes.byref(v) for v in values]))
        return tuple(v.value for v in values)

    @property
    def idle(self) -> bool:
        return bool(self._state()[0])

    @property
    def reserved_pages(self) -> int:
        return self._state()[3]

    @property
    def waiting(self) -> list[Request]:
        count = self._state()[1]
        keys = np.empty(max(1, count), dtype=np.int64)
        host.check(self._lib.hb_sched_waiting_keys(self._handle, host.address(keys), len(keys)))
        return [self.requests[int(k)] for k in keys[:count]]

    # ------------------------------------------------------------------ planning
    def next_plan_arrays(self) -> Optional[PlanArrays]:
        """The next step as arrays, or None when there is nothing to run now (nothing is running or
        waiting, or every running request has its last row in flight)."""
        step, rows, tokens = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        host.check(self._lib.hb_sched_next_plan(self._handle, ctypes.byref(step), ctypes.byref(rows), ctypes.byref(tokens)))
        if step.value < 0:
            return None
        n = rows.value
        plan = PlanArrays(step.value, np.empty(n, np.int64), *[np.empty(n, np.int32) for _ in range(5)], np.empty(tokens.value, np.int32))
        host.check(self._lib.hb_sched_plan(self._handle, plan.step, *[host.address(a) for a in (plan.keys, plan.counts, plan.sample, plan.sampled_before,
                                                                                              plan.from_step, plan.from_index, plan.tokens)]))
        return plan

    def next_plan(self) -> Optional[Plan]:
        arrays = self.next_plan_arrays()
        if arrays is None:
            return None
        rows, at = [], 0
        for i, key in enumerate(arrays.keys.tolist()):
            count = int(arrays.counts[i])
            pending = arrays.from_step[i] >= 0
            rows.append(PlanRow(self.keys.name(key), arrays.tokens[at : at + count].tolist(), bool(arrays.sample[i]), int(arrays.sampled_before[i]),
                                (int(arrays.from_step[i]), int(arrays.from_index[i])) if pending else None))
            at += count
        return Plan(arrays.step, rows)

    # ------------------------------------------------------------------ results
    def complete_arrays(self, step: int, sampled: np.ndarray) -> None:
        """The oldest plan in flight ran: ``sampled`` (int32) holds the token of every sampled row, in row order."""
        sampled = host.ints(sampled)
        host.check(self._lib.hb_sched_complete(self._handle, step, len(sampled), host.address(sampled)))

    def complete(self, plan: Plan, sampled: dict[Hashable, int]) -> list[Event]:
        """The oldest plan in flight ran: ``sampled`` holds the token chosen for every row with ``sample``."""
        self.complete_arrays(plan.step, np.asarray([int(sampled[row.request]) for row in plan.rows if row.sample], dtype=np.int32))
        return self.take_events()

    def fail_step(self, step: int, reason: str) -> None:
        """The step of a plan in flight failed: only the requests it carried fail, and they are released."""
        host.check(self._lib.hb_sched_fail(self._handle, step, reason.encode("utf-8", "replace")))

    def fail(self, plan, reason: str) -> list[Event]:
        self.fail_step(plan.step, reason)
        return self.take_events()

    def cancel(self, request: Hashable) -> bool:
        key = self.keys.known(request)
        if key is None:
            return False
        found = ctypes.c_int()
        host.check(self._lib.hb_sched_cancel(self._handle, key, ctypes.byref(found)))
        return bool(found.value)

    def take_event_arrays(self):
        """(keys, kinds, tokens, reasons) of the events since the last call; kinds index ``EVENT_KINDS``."""
        count, size = ctypes.c_int(), ctypes.c_int()
        host.check(self._lib.hb_sched_take_events(self._handle, 0, None, None, None, None, 0, ctypes.byref(count), ctypes.byref(size)))
        n = count.value
        if n == 0:
            return np.empty(0, np.int64), np.empty(0, np.int32), np.empty(0, np.int32), []
        keys, kinds, tokens = np.empty(n, np.int64), np.empty(n, np.int32), np.empty(n, np.int32)
        text = ctypes.create_string_buffer(max(1, size.value))
        host.check(self._lib.hb_sched_take_events(self._handle, n, host.address(keys), host.address(kinds), host.address(tokens), text, size.value,
                                                  ctypes.byref(count), ctypes.byref(size)))
        reasons = text.raw[: size.value].split(b"\0")[:n]
        return keys, kinds, tokens, [r.decode("utf-8", "replace") for r in reasons]

    def take_events(self) -> list[Event]:
        self._drain_released()  # while the names of requests that just ended are still known
        keys, kinds, tokens, reasons = self.take_event_arrays()
        events = []
        for key, kind, token, reason in zip(keys.tolist(), kinds.tolist(), tokens.tolist(), reasons):
            name = self.keys.name(key)
            if kind == 0:
                events.append(Event(name, "token", token=token))
            else:  # the request's last event: its name and parameters are dropped
                events.append(Event(name, EVENT_KINDS[kind], reason=reason))
                self.requests.pop(key, None)
                self.keys.forget(name)
        return events

    def take_released_keys(self) -> np.ndarray:
        keys, count = np.empty(self.config.max_batch + 1, dtype=np.int64), ctypes.c_int()
        host.check(self._lib.hb_sched_take_released(self._handle, len(keys), host.address(keys), ctypes.byref(count)))
        if count.value > len(keys):  # they stayed queued: again with room
            keys = np.empty(count.value, dtype=np.int64)
            host.check(self._lib.hb_sched_take_released(self._handle, len(keys), host.address(keys), ctypes.byref(count)))
        return keys[: count.value]

    def _drain_released(self) -> None:
        self._released += [self.keys.name(key) for key in self.take_released_keys().tolist()]

    def take_released(self) -> list[Hashable]:
        """Requests whose cache the engine must free (finished, failed or cancelled while running)."""
        self._drain_released()
        released, self._released = self._released, []
        return released
