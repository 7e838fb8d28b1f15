"""The cache manager's accounting and the scheduler's decisions (no GPU)."""
from __future__ import annotations

import random

import pytest

from hyperion_b200.cache import NO_PAGE, CacheError, CacheManager, OutOfPages, PagePool
from hyperion_b200.engine.scheduler import PENDING_TOKEN, Request, Scheduler, SchedulerConfig
from hyperion_b200.parts.base import PagedKV, RequestState
from hyperion_b200.sampling import SamplingParams


def manager(num_pages=8, page_size=4, max_requests=3, window=0):
    users = [(0, PagedKV(2, 16)), (1, PagedKV(2, 16)), (2, PagedKV(2, 16, window=window) if window else PagedKV(2, 16)),
             (3, RequestState((5,)))]
    return CacheManager(users, page_size, num_pages, max_requests)


def test_pool_gives_pages_back_in_fifo_order_and_detects_double_free():
    pool = PagePool(3)
    a, b, c = pool.take(), pool.take(), pool.take()
    assert (a, b, c) == (0, 1, 2) and pool.available == 0
    with pytest.raises(OutOfPages):
        pool.take()
    pool.give_back(b)
    pool.give_back(a)
    with pytest.raises(CacheError):
        pool.give_back(a)
    assert pool.take() == b and pool.take() == a
    pool.check()


def test_groups_by_need():
    m = manager(window=6)
    assert len(m.paged) == 2 and m.paged[0].users == [0, 1] and m.paged[1].users == [2]
    assert m.where(1) == ("paged", 0, 1) and m.where(2) == ("paged", 1, 0) and m.where(3) == ("state", 0, 0)
    same = manager()
    assert len(same.paged) == 1 and same.paged[0].users == [0, 1, 2]


def test_growth_by_pages_and_release_at_the_end():
    m = manager()
    m.add_request("a")
    m.extend("a", 5)
    assert m.table(0, "a") == [0, 1]
    m.advance("a", 5)
    m.extend("a", 3)  # positions 5..7 fit the second page
    assert m.table(0, "a") == [0, 1]
    m.advance("a", 3)
    m.extend("a", 1)
    assert m.table(0, "a") == [0, 1, 2] and m.free_pages() == 5
    m.advance("a", 1)
    m.check()
    m.free("a")
    assert m.free_pages() == 8
    with pytest.raises(CacheError):
        m.free("a")
    m.check()


def test_extend_takes_nothing_when_it_cannot_take_all():
    m = manager(num_pages=4)
    m.add_request("a")
    m.add_request("b")
    m.extend("a", 9)  # 3 pages
    with pytest.raises(OutOfPages):
        m.extend("b", 8)  # needs 2, 1 free
    assert m.table(0, "b") == [] and m.free_pages() == 1
    m.extend_all([("a", 3), ("b", 4)])  # a needs none (positions 9..11 are in its third page), b one
    assert m.free_pages() == 0
    m.check()


def test_extend_all_is_all_or_nothing():
    m = manager(num_pages=4)
    m.add_request("a")
    m.add_request("b")
    with pytest.raises(OutOfPages):
        m.extend_all([("a", 9), ("b", 8)])  # 3 + 2 > 4
    assert m.table(0, "a") == [] and m.table(0, "b") == [] and m.free_pages() == 4
    m.extend_all([("a", 9), ("b", 4)])
    assert m.free_pages() == 0
    m.check()


def test_request_slots_are_bounded_and_reused():
    m = manager(max_requests=2)
    assert m.add_request("a") == 0 and m.add_request("b") == 1
    with pytest.raises(OutOfPages):
        m.add_request("c")
    with pytest.raises(CacheError):
        m.add_request("a")
    m.free("a")
    assert m.add_request("c") == 0
    m.check()


def test_window_group_gives_pages_back_while_the_request_lives():
    m = manager(num_pages=6, page_size=4, window=6)
    m.add_request("a")
    full, windowed = 0, 1
    for step in range(20):
        m.extend("a", 1)
        m.advance("a", 1)
        m.check()
    # length 20: the next query (position 20) reads keys 15..20, so blocks 0..2 (positions 0..11) are gone
    assert m.table(windowed, "a")[:3] == [NO_PAGE] * 3 and all(p != NO_PAGE for p in m.table(windowed, "a")[3:])
    assert all(p != NO_PAGE for p in m.table(full, "a")) and len(m.table(full, "a")) == 5
    assert m.free_pages(windowed) == 6 - 2
    # a long portion needs pages for all its positions during the step and gives most back after it
    m.add_request("b")
    with pytest.raises(OutOfPages):
        m.extend("b", 17)  # 5 pages, the full group has 1 free
    m.free("a")
    m.extend("b", 17)
    m.advance("b", 17)
    assert m.free_pages(windowed) == 6 - 2
    m.check()


def test_random_orders_never_lose_or_share_a_page():
    rng = random.Random(7)
    m = manager(num_pages=24, page_size=4, max_requests=5, window=10)
    live: dict[str, int] = {}
    counter = 0
    for _ in range(2000):
        action = rng.random()
        if action < 0.2 and len(live) < 5:
            name = f"r{counter}"
            counter += 1
            m.add_request(name)
            live[name] = 0
        elif action < 0.85 and live:
            name = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 13])
            try:
                m.extend(name, n)
                m.advance(name, n)
                live[name] += n
                assert m.length(name) == live[name]
            except OutOfPages:
                pass
        elif live:
            name = rng.choice(list(live))
            m.free(name)
            del live[name]
        m.check()
    for name in list(live):
        m.free(name)
    m.check()
    assert all(m.free_pages(g) == 24 for g in range(len(m.paged)))


# ---------------------------------------------------------------------------------- scheduler
def params(max_tokens=4, **kw):
    return SamplingParams(temperature=0.0, max_tokens=max_tokens, **kw).validated()


def drive(scheduler, token_of=lambda request, n: 100 + n, limit=1000):
    """Run plans to the end with a stub that 'samples' token_of(request, count so far)."""
    plans, events = [], []
    counts: dict = {}
    for _ in range(limit):
        plan = scheduler.next_plan()
        events += scheduler.take_events()
        if plan is None:
            assert scheduler.idle
            return plans, events
        plans.append(plan)
        sampled = {}
        for row in plan.rows:
            if row.sample:
                counts[row.request] = counts.get(row.request, 0) + 1
                sampled[row.request] = token_of(row.request, counts[row.request])
        events += scheduler.complete(plan, sampled)
    raise AssertionError("the scheduler did not finish")


def test_prompt_is_cut_under_the_token_budget_then_decoded():
    s = Scheduler(SchedulerConfig(num_pages=100, page_size=4, max_seq_len=64, max_batch_tokens=8))
    s.enqueue(Request("a", list(range(19)), params(3)))
    plans, events = drive(s)
    assert [len(p.rows[0].tokens) for p in plans] == [8, 8, 3, 1, 1]
    assert [p.rows[0].sample for p in plans] == [False, False, True, True, True]
    assert [e.token for e in events if e.kind == "token"] == [101, 102, 103]
    assert events[-1].kind == "finished" and events[-1].reason == "length"
    assert s.take_released() == ["a"]


def test_decode_rows_ride_with_prompt_portions_limited_while_busy():
    s = Scheduler(SchedulerConfig(num_pages=100, page_size=4, max_seq_len=128, max_batch_tokens=16, prefill_chunk_busy=5))
    s.enqueue(Request("a", list(range(6)), params(10)))
    first = s.next_plan()
    s.complete(first, {"a": 50})
    s.enqueue(Request("b", list(range(20)), params(2)))
    plan = s.next_plan()
    assert [(r.request, len(r.tokens), r.sample) for r in plan.rows] == [("a", 1, True), ("b", 5, False)]
    assert plan.rows[0].tokens == [50] and plan.rows[0].sampled_before == 1
    s.complete(plan, {"a": 51})
    plan = s.next_plan()
    assert [(r.request, len(r.tokens)) for r in plan.rows] == [("a", 1), ("b", 5)]


def test_oldest_prompt_first_and_budget_shared():
    s = Scheduler(SchedulerConfig(num_pages=100, page_size=4, max_seq_len=128, max_batch_tokens=10))
    s.enqueue(Request("a", list(range(7)), params()))
    s.enqueue(Request("b", list(range(7)), params()))
    plan = s.next_plan()
    assert [(r.request, len(r.tokens), r.sample) for r in plan.rows] == [("a", 7, True), ("b", 3, False)]


def test_eos_ends_a_request_without_emitting_it_unless_ignored():
    config = SchedulerConfig(num_pages=100, page_size=4, max_seq_len=64, eos_token_ids=(9,))
    s = Scheduler(config)
    s.enqueue(Request("a", [1, 2], params(10)))
    _, events = drive(s, token_of=lambda r, n: 9 if n == 3 else 5)
    assert [e.token for e in events if e.kind == "token"] == [5, 5] and events[-1].reason == "stop"
    s = Scheduler(config)
    s.enqueue(Request("a", [1, 2], params(4, ignore_eos=True)))
    _, events = drive(s, token_of=lambda r, n: 9)
    assert [e.token for e in events if e.kind == "token"] == [9, 9, 9, 9] and events[-1].reason == "length"


def test_context_limit_ends_with_length():
    s = Scheduler(SchedulerConfig(num_pages=100, page_size=4, max_seq_len=8))
    s.enqueue(Request("a", [1, 2, 3, 4, 5], params(100)))
    _, events = drive(s)
    assert len([e for e in events if e.kind == "token"]) == 3 and events[-1].reason == "length"


def test_admission_reserves_the_worst_case_and_waits_for_pages():
    # 6 pages of 4 tokens; each request needs ceil((6 + 6) / 4) = 3 pages: two run, the third waits
    s = Scheduler(SchedulerConfig(num_pages=6, page_size=4, max_seq_len=64, max_batch_tokens=64))
    for name in "abc":
        s.enqueue(Request(name, list(range(6)), params(6)))
    plan = s.next_plan()
    assert [r.request for r in plan.rows] == ["a", "b"] and s.reserved_pages == 6 and len(s.waiting) == 1
    plans, events = [plan], []
    events += s.complete(plan, {"a": 1, "b": 1})
    more, later = drive(s)
    started = next(i for i, p in enumerate(more) if any(r.request == "c" for r in p.rows))
    finished_before = [e.request for e in events + later if e.kind == "finished"]
    assert set(finished_before) == {"a", "b", "c"}
    # c started only after a or b had finished
    assert all(all(r.request != "c" for r in p.rows) for p in more[:started])
    assert s.idle


def test_a_request_that_can_never_fit_fails_at_once_and_others_go_on():
    s = Scheduler(SchedulerConfig(num_pages=4, page_size=4, max_seq_len=64))
    s.enqueue(Request("big", list(range(30)), params(4)))
    s.enqueue(Request("empty", [], params(4)))
    s.enqueue(Request("ok", [1, 2, 3], params(2)))
    plans, events = drive(s)
    failed = {e.request: e.reason for e in events if e.kind == "failed"}
    assert "needs 9 pages, the pool has 4" in failed["big"] and "empty" in failed
    assert [e.token for e in events if e.kind == "token" and e.request == "ok"] == [101, 102]


def test_cancel_and_fail_release_only_their_requests():
    s = Scheduler(SchedulerConfig(num_pages=100, page_size=4, max_seq_len=64))
    s.enqueue(Request("a", [1, 2, 3], params(5)))
    s.enqueue(Request("b", [4, 5], params(5)))
    plan = s.next_plan()
    s.complete(plan, {"a": 7, "b": 8})
    assert s.cancel("a") and not s.cancel("zzz")
    assert s.take_released() == ["a"]
    plan = s.next_plan()
    assert [r.request for r in plan.rows] == ["b"]
    events = s.fail(plan, "device error")
    assert [(e.request, e.kind) for e in events if e.kind == "failed"] == [("b", "failed")]
    assert s.take_released() == ["b"] and s.idle


def test_same_trace_gives_the_same_plans():
    def run():
        s = Scheduler(SchedulerConfig(num_pages=40, page_size=4, max_seq_len=64, max_batch_tokens=12, prefill_chunk_busy=4, max_batch=3))
        for i, n in enumerate([9, 17, 3, 25, 6]):
            s.enqueue(Request(i, list(range(n)), params(3 + i)))
        plans, _ = drive(s)
        return [[(r.request, tuple(r.tokens), r.sample, r.sampled_before) for r in p.rows] for p in plans]

    assert run() == run()


# ---------------------------------------------------------------------- plans that run ahead of their results
def drive_ahead(scheduler, token_of, limit=1000):
    """Like ``drive`` but each plan is made before the one before it is completed, as a pipelined
    engine does; a pending token is resolved from the plan it names, which must be the one before."""
    events, in_flight, tokens_of_plan = [], [], {}
    fed: dict = {}  # request -> the tokens its rows carried, pending ones resolved
    counts: dict = {}
    for _ in range(limit):
        plan = scheduler.next_plan() if len(in_flight) < 2 else None
        events += scheduler.take_events()
        if plan is not None:
            sampled = {}
            for row in plan.rows:
                tokens = row.tokens
                if row.token_from is not None:
                    step, index = row.token_from
                    assert tokens == [PENDING_TOKEN] and step == plan.step - 1
                    tokens = [tokens_of_plan[step][index]]
                else:
                    assert PENDING_TOKEN not in tokens
                fed.setdefault(row.request, []).extend(tokens)
                if row.sample:
                    counts[row.request] = counts.get(row.request, 0) + 1
                    assert row.sampled_before == counts[row.request] - 1
                    sampled[row.request] = token_of(row.request, counts[row.request])
            tokens_of_plan[plan.step] = [sampled[row.request] for row in plan.rows if row.sample]
            in_flight.append((plan, sampled))
        if in_flight and (plan is None or len(in_flight) >= 2):
            events += scheduler.complete(*in_flight.pop(0))
        elif plan is None:
            assert scheduler.idle
            return events, fed
    raise AssertionError("the scheduler did not finish")


def outcome(events):
    tokens, reasons = {}, {}
    for e in events:
        if e.kind == "token":
            tokens.setdefault(e.request, []).append(e.token)
        else:
            reasons[e.request] = (e.kind, e.reason)
    return tokens, reasons


def test_plans_ahead_of_results_give_the_same_tokens_and_reasons():
    eos = 7

    def token_of(request, n):  # request 2 and 5 meet the end-of-sequence token, the others end by length
        return eos if request in (2, 5) and n == request else 100 + 10 * request + n

    def scheduler(depth):
        s = Scheduler(SchedulerConfig(num_pages=40, page_size=4, max_seq_len=48, max_batch=3, max_batch_tokens=12, prefill_chunk_busy=5,
                                      eos_token_ids=(eos,), max_in_flight=depth))
        r = random.Random(6)
        for i in range(8):
            s.enqueue(Request(i, [r.randrange(50) for _ in range(r.randrange(1, 30))], params(2 + (5 * i) % 9)))
        return s

    _, events = drive(scheduler(1), token_of)
    ahead_events, fed = drive_ahead(scheduler(2), token_of)
    assert outcome(ahead_events) == outcome(events)
    tokens, reasons = outcome(events)
    assert reasons[2] == ("finished", "stop") and reasons[5] == ("finished", "stop") and reasons[0] == ("finished", "length")
    reference = scheduler(1)
    for request in list(reference.waiting):  # every request was fed its prompt, then its own tokens, nothing else
        generated = tokens.get(request.id, [])
        carried = fed[request.id]
        assert carried[: len(request.prompt)] == list(request.prompt)
        extra = carried[len(request.prompt):]
        assert extra[: len(generated)] == generated[: len(extra)] and len(extra) <= len(generated) + 1


def test_no_row_is_planned_past_max_tokens_or_the_context_limit_when_running_ahead():
    s = Scheduler(SchedulerConfig(num_pages=100, page_size=4, max_seq_len=10, max_batch_tokens=64, max_in_flight=2))
    s.enqueue(Request("a", list(range(4)), params(2)))
    s.enqueue(Request("b", list(range(7)), params(50)))
    first = s.next_plan()
    second = s.next_plan()  # both decode from the device
    assert [(r.request, r.tokens, r.token_from) for r in second.rows] == [("a", [PENDING_TOKEN], (0, 0)), ("b", [PENDING_TOKEN], (0, 1))]
    with pytest.raises(RuntimeError):
        s.next_plan()
    s.complete(first, {"a": 11, "b": 21})
    third = s.next_plan()  # a has its two rows; b may take one more (7 + 3 = 10 is the limit)
    assert [(r.request, r.token_from) for r in third.rows] == [("b", (1, 1))]
    s.complete(second, {"a": 12, "b": 22})
    assert s.next_plan() is None and not s.idle  # b's last row is in flight: nothing to plan, not idle
    events = s.complete(third, {"b": 23})
    assert [e.token for e in events if e.kind == "token"] == [23] and events[-1].reason == "length"
    assert s.idle


def test_a_known_token_is_fed_from_the_host_even_with_room_to_run_ahead():
    s = Scheduler(SchedulerConfig(num_pages=100, page_size=4, max_seq_len=64, max_in_flight=2))
    s.enqueue(Request("a", [1, 2, 3], params(4)))
    first = s.next_plan()
    s.complete(first, {"a": 9})
    assert s.next_plan().rows[0].tokens == [9]


# ---------------------------------------------------------------------- step assembly by the host runtime
def test_step_assembly_writes_every_array_where_its_layout_says():
    import numpy as np
    import torch

    from hyperion_b200.engine.batch import MetadataPacker

    users = [(0, PagedKV(2, 16, 0)), (1, PagedKV(2, 16, 10))]
    m = CacheManager(users, page_size=4, num_pages=32, max_requests=4)
    for name, tokens in (("a", 9), ("b", 3), ("c", 17)):
        m.add_request(name)
        m.extend(name, tokens)
        m.advance(name, tokens)
    work = [("c", 2), ("a", 1), ("b", 6)]  # c and a decode or continue, b brings a portion
    m.extend_all(work)
    keys = np.asarray([m.keys.known(name) for name, _ in work], dtype=np.int64)
    counts = np.asarray([n for _, n in work], dtype=np.int32)
    tokens = np.arange(100, 109, dtype=np.int32)
    want = np.asarray([1, 2, 8], dtype=np.int32)
    packer = MetadataPacker(torch.device("cpu"), capacity=64)  # too small on purpose: it grows and keeps what was written
    packer.begin()
    packer.add("before", [7, 7, 7])
    packer.add_step(m, keys, counts, tokens, want, table_step=0)
    packer.add("after", [5])
    arrays = {name: value.clone() for name, value in packer.finish().items()}
    assert arrays["before"].tolist() == [7, 7, 7] and arrays["after"].tolist() == [5]
    assert arrays["token_ids"].tolist() == tokens.tolist()
    assert arrays["positions"].tolist() == [17, 18, 9, 3, 4, 5, 6, 7, 8]
    assert arrays["token_row"].tolist() == [0, 0, 1, 2, 2, 2, 2, 2, 2]
    assert arrays["row_start"].tolist() == [0, 2, 3, 9]
    assert arrays["slots"].tolist() == [m.slot("c"), m.slot("a"), m.slot("b")]
    assert arrays["want"].tolist() == [1, 2, 8]
    for group in (0, 1):
        tables = [m.table(group, name) for name, _ in work]
        width = max(len(t) for t in tables)
        assert arrays[f"table{group}"].tolist() == [t + [NO_PAGE] * (width - len(t)) for t in tables]
    assert NO_PAGE in m.table(1, "c")  # the window of group 1 has passed c's first pages: they read as missing in the step too
    assert all(start % 4 == 0 for _, start, _, _ in packer._items)
    # widths of a graphed decode step are padded to whole steps
    packer.begin()
    packer.add_step(m, keys, np.ones(3, np.int32), tokens[:3], np.arange(3, dtype=np.int32), table_step=8)
    assert packer.finish()["table0"].shape == (3, 8)


def test_step_assembly_refuses_what_it_cannot_place():
    import numpy as np
    import torch

    from hyperion_b200.engine.batch import MetadataPacker

    m = manager()
    m.add_request("a")
    m.extend("a", 2)
    packer = MetadataPacker(torch.device("cpu"), capacity=64)
    packer.begin()
    keys, one = np.asarray([m.keys.known("a")], np.int64), np.ones(1, np.int32)
    with pytest.raises(ValueError):
        packer.add_step(m, keys, one, one, np.asarray([3], np.int32), 0)  # a wanted place beyond the tokens
    with pytest.raises(CacheError):
        packer.add_step(m, np.asarray([12345], np.int64), one, one, np.empty(0, np.int32), 0)  # a request the cache does not know


def test_attention_plan_cuts_long_rows_into_tiles_and_leaves_short_rows_as_items():
    from hyperion_b200.engine.batch import Row
    from hyperion_b200.ops import attention

    rows, start = [], 0
    for count in (1, 40, 4, 5, 16):
        rows.append(Row("r", start, count, 0, 0))
        start += count
    tiles, items = attention.plan(rows, 16)
    assert items.tolist() == [0, 41, 42, 43, 44]
    assert tiles.reshape(-1, 3).tolist() == [[1, 16, 1], [17, 16, 1], [33, 8, 1], [45, 5, 3], [50, 16, 4]]


def test_released_requests_are_not_lost_when_many_end_at_once():
    s = Scheduler(SchedulerConfig(num_pages=1000, page_size=4, max_seq_len=64, max_batch=2, max_batch_tokens=64))
    for i in range(7):
        s.enqueue(Request(i, [1, 2], params(1)))
    import numpy as np

    while (plan := s.next_plan_arrays()) is not None:  # nobody takes events or released requests meanwhile: more pile up than run at a time
        s.complete_arrays(plan.step, np.full(int(plan.sample.sum()), 5, np.int32))
    assert sorted(s.take_released()) == list(range(7)) and s.take_released() == []
    assert [e.kind for e in s.take_events()].count("finished") == 7


def test_cancel_and_fail_while_plans_run_ahead():
    s = Scheduler(SchedulerConfig(num_pages=100, page_size=4, max_seq_len=64, max_batch_tokens=64, max_in_flight=2))
    for name in "abc":
        s.enqueue(Request(name, [1, 2, 3], params(6)))
    first = s.next_plan()   # three prompts, three samples
    second = s.next_plan()  # three decode rows fed from the device
    assert [r.token_from for r in second.rows] == [(0, 0), (0, 1), (0, 2)]
    assert s.cancel("b")  # while both plans are in flight
    events = s.complete(first, {"a": 10, "b": 11, "c": 12})
    assert [(e.request, e.kind, e.token) for e in events if e.kind == "token"] == [("a", "token", 10), ("c", "token", 12)]
    assert ("b", "finished", "cancelled") in [(e.request, e.kind, e.reason) for e in events]
    third = s.next_plan()  # b is gone; a and c still feed from the device (plan 1 is in flight)
    assert [(r.request, r.token_from) for r in third.rows] == [("a", (1, 0)), ("c", (1, 2))]
    events = s.fail(second, "KernelError: boom")  # the older plan in flight fails: its requests fail and are released
    assert sorted((e.request, e.kind) for e in events) == [("a", "failed"), ("c", "failed")]
    assert sorted(s.take_released()) == ["a", "b", "c"]
    assert s.complete(third, {"a": 1, "c": 2}) == []  # rows of requests that are gone are dropped
    assert s.idle and s.next_plan() is None


def test_enqueue_refuses_a_known_id_and_a_full_queue():
    from hyperion_b200.host import QueueFull

    s = Scheduler(SchedulerConfig(num_pages=100, page_size=4, max_seq_len=64, max_queue=2))
    s.enqueue(Request("a", [1], params(1)))
    with pytest.raises(ValueError):
        s.enqueue(Request("a", [2], params(1)))
    s.enqueue(Request("b", [1], params(1)))
    with pytest.raises(QueueFull):
        s.enqueue(Request("c", [1], params(1)))
    drive(s)
    s.enqueue(Request("a", [3], params(1)))  # a finished: its name may come again


# ---------------------------------------------------------------------- sizes at the edge, turns, and groups of the cache
def test_a_huge_max_tokens_is_reserved_in_64_bits_and_capped_by_the_context():
    """prompt + max_tokens passes 2^31: the need is the context limit's, never negative, and the next request still waits."""
    s = Scheduler(SchedulerConfig(num_pages=8, page_size=4, max_seq_len=32, max_batch_tokens=64))
    s.enqueue(Request("big", list(range(6)), params(2**31 - 1)))
    s.enqueue(Request("next", list(range(6)), params(100000)))
    plan = s.next_plan()
    assert [r.request for r in plan.rows] == ["big"]
    assert s.reserved_pages == 8 and len(s.waiting) == 1  # 32 tokens of context = 8 pages: the pool is spoken for
    with pytest.raises(Exception, match="max_tokens"):
        SamplingParams(max_tokens=2**31).validated()
    with pytest.raises(ValueError, match="max_tokens"):
        s.enqueue(Request("over", [1], SamplingParams(temperature=0.0, max_tokens=2**31)))  # not validated by the caller


def test_more_decoding_requests_than_the_budget_take_turns():
    """6 requests decode under a budget of 4 tokens: nobody waits longer than one step, prompts that wait keep half of the
    budget, and a second run repeats the plans (the reference's round robin, helios/crates/helios-core/src/step_scheduler.rs:273-289)."""
    def run():
        s = Scheduler(SchedulerConfig(num_pages=100, page_size=4, max_seq_len=64, max_batch_tokens=4, prefill_chunk_busy=4))
        for name in "abcdef":
            s.enqueue(Request(name, [1], params(5)))
        plans, events = drive(s)
        return s, plans, events

    s, plans, events = run()
    rows = [[(r.request, r.sampled_before > 0) for r in p.rows] for p in plans]
    assert all(sum(len(r.tokens) for r in p.rows) <= 4 for p in plans)
    assert rows[0] == [(n, False) for n in "abcd"]  # four prompts of one token
    assert rows[1] == [("a", True), ("b", True), ("e", False), ("f", False)]  # the prompts that wait keep half of the budget
    assert rows[2] == [(n, True) for n in "cdef"]  # c and d were left out: they lead now
    assert rows[3] == [(n, True) for n in "abcd"] and rows[4] == [(n, True) for n in "abef"]
    assert all(p == sorted(p) for p in rows)  # admission order inside a plan
    waited = {name: 0 for name in "abcdef"}
    left = {name: 5 for name in "abcdef"}
    for plan in rows[2:]:
        for name in [n for n in "abcdef" if left[n] > 0]:
            if any(r == name for r, _ in plan):
                waited[name], left[name] = 0, left[name] - 1
            else:
                waited[name] += 1
                assert waited[name] <= 1, (name, rows)
    tokens = {name: [e.token for e in events if e.kind == "token" and e.request == name] for name in "abcdef"}
    assert all(len(t) == 5 for t in tokens.values()) and s.idle
    again = run()[1]
    assert [[(r.request, tuple(r.tokens)) for r in p.rows] for p in again] == [[(r.request, tuple(r.tokens)) for r in p.rows] for p in plans]


def test_turns_go_on_when_a_request_in_front_of_the_cursor_ends():
    s = Scheduler(SchedulerConfig(num_pages=100, page_size=4, max_seq_len=64, max_batch_tokens=2, prefill_chunk_busy=2))
    lengths = dict(zip("abcd", (2, 6, 6, 6)))
    for name, n in lengths.items():
        s.enqueue(Request(name, [1], params(n)))
    plans, events = drive(s)
    rows = [[r.request for r in p.rows] for p in plans]
    left, waited = dict(lengths), {name: 0 for name in lengths}
    for step in rows:
        for name in [n for n in lengths if left[n] > 0]:
            if name in step:
                waited[name], left[name] = 0, left[name] - 1
            else:
                waited[name] += 1
                assert waited[name] <= 3, (name, rows)  # at most the others' turns: 4 requests, 2 rows a step, prompts keep one
    assert s.idle and all(len([e for e in events if e.kind == "token" and e.request == name]) == n for name, n in lengths.items())


def test_worst_case_pages_bounds_what_a_windowed_request_ever_holds():
    """Random portions through a windowed group: the pages held at any moment never pass the bound admission reserves."""
    import ctypes

    from hyperion_b200 import host

    def bound(page, window, tokens, portion):
        value = ctypes.c_int()
        host.check(host.library().hb_cache_worst_case_pages(page, window, tokens, portion, ctypes.byref(value)))
        return value.value

    assert bound(4, 0, 33, 7) == 9 and bound(4, 6, 5, 100) == 2 and bound(16, 0, 0, 1) == 0
    rng = random.Random(5)
    for _ in range(60):
        page = rng.choice([1, 2, 4, 8, 16])
        window = rng.randint(1, 40)
        portion = rng.randint(1, 30)
        total = rng.randint(1, 200)
        m = CacheManager([(0, PagedKV(1, 8, window=window))], page, 400, 1)
        m.add_request("r")
        limit, fed, most = bound(page, window, total, portion), 0, 0
        while fed < total:
            n = min(rng.randint(1, portion), total - fed)
            m.extend("r", n)
            most = max(most, 400 - m.free_pages(0))
            m.advance("r", n)
            fed += n
        assert most <= limit, (page, window, portion, total, most, limit)
        m.free("r")


def test_admission_counts_pages_per_group_of_the_cache():
    # a windowed group: the window (8) and one portion (4) span ceil(11 / 4) + 1 = 4 pages however long the request gets
    s = Scheduler(SchedulerConfig(num_pages=8, page_size=4, max_seq_len=1000, max_batch_tokens=4, group_windows=(8,)))
    for name in "abc":
        s.enqueue(Request(name, list(range(30)), params(500)))
    s.next_plan()
    assert s.reserved_pages == 8 and len(s.waiting) == 1  # two run although each will pass 500 tokens
    # the same requests with a group that keeps every key beside it: that group decides
    s = Scheduler(SchedulerConfig(num_pages=8, page_size=4, max_seq_len=1000, max_batch_tokens=4, group_windows=(8, 0)))
    s.enqueue(Request("a", list(range(30)), params(500)))
    s.next_plan()
    assert any(e.kind == "failed" and "needs 133 pages" in e.reason for e in s.take_events())
    # no paged group at all (a model of fixed per-request state only): pages are not asked for, the request slots decide
    s = Scheduler(SchedulerConfig(num_pages=1, page_size=4, max_seq_len=1000, max_batch=2, max_batch_tokens=64, group_windows=()))
    for name in "abc":
        s.enqueue(Request(name, list(range(30)), params(500)))
    plan = s.next_plan()
    assert [r.request for r in plan.rows] == ["a", "b"] and s.reserved_pages == 0 and len(s.waiting) == 1


def test_a_cache_user_may_keep_any_payload_of_fixed_shape_per_token():
    from hyperion_b200.parts.base import PagedTokens

    latent = PagedTokens(inner=(24,))
    m = CacheManager([(0, PagedKV(2, 16)), (1, latent), (2, latent), (3, PagedTokens(outer=(3,), inner=(2, 5), window=9))], 4, 8, 2)
    assert [g.users for g in m.paged] == [[0], [1, 2], [3]] and m.group_windows == [0, 0, 9]
    assert m.bytes_per_token() == (2 * 2 * 16 + 2 * 24 + 3 * 2 * 5) * 4  # float32 by default
    assert latent.storage_shape(8, 4) == (8, 4, 24) and PagedKV(2, 16).storage_shape(8, 4) == (8, 2, 2, 4, 16)
