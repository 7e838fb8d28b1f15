"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
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
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Hashable, Optional, Sequence, Union

from ..sampling.params import SamplingParams


PENDING_TOKEN = -1  # stands in a plan row for a sampled token that has not reached the host yet


class QueueFull(RuntimeError):
    pass


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
class Event:
    request: Hashable
    kind: str  # "token" | "finished" | "failed"
    token: Optional[int] = None
    reason: Optional[str] = None  # "stop" | "length" | "cancelled" | message of a failure


@dataclass
class _Sequence:
    request: Request
    reserved_pages: int
    fed: int = 0  # prompt tokens already planned
    planned_samples: int = 0  # sampled rows planned so far, results in or not
    generated: list[int] = field(default_factory=list)
    feed: Union[None, int, tuple[int, int]] = None  # what the next decode row feeds: a token, or where a plan in flight will put it

    @property
    def prefilling(self) -> bool:
        return self.fed < len(self.request.prompt)


class Scheduler:
    def __init__(self, config: SchedulerConfig):
        if config.max_batch_tokens < 1 or config.prefill_chunk_busy < 1 or config.max_batch < 1:
            raise ValueError("max_batch_tokens, prefill_chunk_busy and max_batch must be at least 1")
        self.config = config
        self.waiting: deque[Request] = deque()
        self.running: dict[Hashable, _Sequence] = {}  # insertion order = admission order
        self.events: list[Event] = []
        self.released: list[Hashable] = []  # requests whose cache the engine must free
        self._step = 0
        self._in_flight: deque[Plan] = deque()  # oldest first

    # ------------------------------------------------------------------ intake
    def enqueue(self, request: Request) -> None:
        if len(self.waiting) >= self.config.max_queue:
            raise QueueFull(f"{len(self.waiting)} requests are waiting")
        if request.id in self.running or any(r.id == request.id for r in self.waiting):
            raise ValueError(f"request id {request.id!r} is already known")
        self.waiting.append(request)

    def _pages(self, tokens: int) -> int:
        return -(-tokens // self.config.page_size)

    @property
    def reserved_pages(self) -> int:
        return sum(s.reserved_pages for s in self.running.values())

    def _admit(self) -> None:
        c = self.config
        while self.waiting and len(self.running) < c.max_batch:
            request = self.waiting[0]
            prompt = len(request.prompt)
            if prompt == 0 or prompt >= c.max_seq_len:
                self.waiting.popleft()
                self.events.append(Event(request.id, "failed", reason=f"prompt of {prompt} tokens is outside 1..{c.max_seq_len - 1}"))
                continue
            need = self._pages(min(prompt + request.params.max_tokens, c.max_seq_len))
            if need > c.num_pages:
                self.waiting.popleft()
                self.events.append(Event(request.id, "failed", reason=f"needs {need} pages, the pool has {c.num_pages}"))
                continue
            if self.reserved_pages + need > c.num_pages:
                return  # waits for running requests to finish; order is kept
            self.waiting.popleft()
            self.running[request.id] = _Sequence(request, need)

    # ------------------------------------------------------------------ planning
    def next_plan(self) -> Optional[Plan]:
        """The next step, or None when there is nothing to run now (nothing is running or waiting,
        or every running request has its last row in flight)."""
        if len(self._in_flight) >= self.config.max_in_flight:
            raise RuntimeError("the previous plan has not been completed")
        self._admit()
        c = self.config
        rows: list[PlanRow] = []
        budget = c.max_batch_tokens
        decoding = [s for s in self.running.values() if s.feed is not None]
        for s in decoding:
            if budget == 0:
                break
            if isinstance(s.feed, tuple):
                rows.append(PlanRow(s.request.id, [PENDING_TOKEN], True, s.planned_samples, token_from=s.feed))
            else:
                rows.append(PlanRow(s.request.id, [s.feed], True, s.planned_samples))
            budget -= 1
        limit = c.prefill_chunk_busy if decoding else c.max_batch_tokens
        for s in self.running.values():
            if budget == 0:
                break
            if not s.prefilling:
                continue
            prompt = s.request.prompt
            count = min(len(prompt) - s.fed, budget, limit)
            rows.append(PlanRow(s.request.id, list(prompt[s.fed : s.fed + count]), s.fed + count == len(prompt), 0))
            s.fed += count
            budget -= count
        if not rows:
            return None
        sampled = 0
        for row in rows:  # what each request feeds next is known now, but for the token's value
            if not row.sample:
                continue
            s = self.running[row.request]
            s.planned_samples += 1
            more = s.planned_samples < s.request.params.max_tokens and len(s.request.prompt) + s.planned_samples < c.max_seq_len
            s.feed = (self._step, sampled) if more else None
            sampled += 1
        plan = Plan(self._step, rows)
        self._step += 1
        self._in_flight.append(plan)
        return plan

    # ------------------------------------------------------------------ results
    def complete(self, plan: Plan, sampled: dict[Hashable, int]) -> list[Event]:
        """The oldest plan in flight ran: ``sampled`` holds the token chosen for every row with ``sample``."""
        if not self._in_flight or plan is not self._in_flight[0]:
            raise RuntimeError("complete() must get the oldest plan in flight")
        self._in_flight.popleft()
        c = self.config
        index = -1
        for row in plan.rows:
            if not row.sample:
                continue
            index += 1
            s = self.running.get(row.request)
            if s is None:  # cancelled, or ended by an end-of-sequence token, while this row was in flight
                continue
            token = int(sampled[row.request])
            params = s.request.params
            if token in c.eos_token_ids and not params.ignore_eos:
                self._finish(s, "stop")
                continue
            s.generated.append(token)
            self.events.append(Event(row.request, "token", token=token))
            if len(s.generated) >= params.max_tokens or len(s.request.prompt) + len(s.generated) >= c.max_seq_len:
                self._finish(s, "length")
            elif s.feed == (plan.step, index):
                s.feed = token  # no later plan has taken it from the device
        return self.take_events()

    def fail(self, plan: Plan, reason: str) -> list[Event]:
        """The step failed: only the requests it carried fail, and they are released."""
        if plan not in self._in_flight:
            raise RuntimeError("fail() must get a plan in flight")
        self._in_flight.remove(plan)
        for row in plan.rows:
            s = self.running.pop(row.request, None)
            if s is not None:
                self.released.append(row.request)
                self.events.append(Event(row.request, "failed", reason=reason))
        return self.take_events()

    def cancel(self, request: Hashable) -> bool:
        for index, waiting in enumerate(self.waiting):
            if waiting.id == request:
                del self.waiting[index]
                self.events.append(Event(request, "finished", reason="cancelled"))
                return True
        s = self.running.pop(request, None)
        if s is None:
            return False
        self.released.append(request)
        self.events.append(Event(request, "finished", reason="cancelled"))
        return True

    def _finish(self, s: _Sequence, reason: str) -> None:
        del self.running[s.request.id]
        self.released.append(s.request.id)
        self.events.append(Event(s.request.id, "finished", reason=reason))

    def take_events(self) -> list[Event]:
        events, self.events = self.events, []
        return events

    def take_released(self) -> list[Hashable]:
        released, self.released = self.released, []
        return released

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running
