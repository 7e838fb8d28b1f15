"""Trace replay on the GPU: the same requests whole, with the last 32 tokens one by one, in portions
of changing size, and mixed with other requests over a pool so small that pages are reused; in
float32 and in bfloat16, every position compared with the plain implementation."""
from __future__ import annotations

import numpy as np
import pytest

from helpers import TINY, TOLERANCE, check_pages_log, compare_steps, logits_by_position, make_folder, plain_logits, random_ids, run_trace

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 45, 100, 33, 90, 61], "B": [130, 40, 77, 200, 35, 96], "C": [150, 37, 66, 210, 80, 129]}


def requests_for(name: str) -> dict[str, list[int]]:
    config, seed = TINY[name]
    return {f"r{i}": random_ids(100 * seed + i, n, config.vocab_size) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module", params=["A", "B", "C"])
def model(request, tmp_path_factory):
    name = request.param
    folder = make_folder(tmp_path_factory.mktemp(f"model_{name}"), name)
    requests = requests_for(name)
    reference = {rid: plain_logits(folder, ids) for rid, ids in requests.items()}
    return name, folder, requests, reference


def round64(n: int) -> int:
    return -(-n // 64) * 64


def whole_steps(requests):
    steps = []
    for i, (rid, ids) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]})
    return steps


def tail_steps(requests, tail=32):
    steps = []
    for rid, ids in requests.items():
        head = len(ids) - tail
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[:head], "want": [head - 1]}], "end": []})
        for k in range(head, len(ids)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [ids[k]], "want": [0]}],
                          "end": [rid] if k == len(ids) - 1 else []})
    return steps


def portion_steps(requests, sizes=(7, 2, 16, 3, 2, 33, 5, 2, 64, 9)):
    steps = []
    k = 0
    for rid, ids in requests.items():
        at = 0
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            if len(ids) - at - n == 1:  # never leave a single token over: portions go down to two
                n += 1
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[at:at + n], "want": list(range(n))}],
                          "end": [rid] if at + n == len(ids) else []})
            at += n
    return steps


def mixed_steps(requests, live_max=4, decode_tail=12, sizes=(5, 2, 19, 3, 8, 2, 30, 4)):
    """Up to four live requests; portions of some beside single tokens of others; a request sits out
    every fifth step; new requests start as others end, so freed pages go to later requests."""
    waiting = list(requests.items())
    live: dict[str, int] = {}
    steps = []
    peak = 0
    k = 0
    while waiting or live:
        while waiting and len(live) < live_max:
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, ended = [], []
        for j, rid in enumerate(list(live)):
            ids, at = requests[rid], live[rid]
            if (len(steps) + j) % 5 == 4 and len(live) > 1:
                continue
            n = 1 if at >= len(ids) - decode_tail else min(sizes[k % len(sizes)], len(ids) - decode_tail - at)
            k += 1
            entries.append({"id": rid, "tokens": ids[at:at + n], "want": list(range(n))})
            live[rid] = at + n
            if live[rid] == len(ids):
                ended.append(rid)
        peak = max(peak, sum(round64(at) for at in live.values()))
        steps.append({"step": len(steps), "entries": entries, "end": ended})
        for rid in ended:
            del live[rid]
    return steps, peak


DRIVES = ("whole", "last32", "portions", "mixed")


def drive_steps(requests, drive):
    """(steps, --max-tokens) of one of the four ways of cutting the same requests."""
    longest = round64(max(map(len, requests.values())))
    if drive == "whole":
        return whole_steps(requests), longest
    if drive == "last32":
        return tail_steps(requests), longest
    if drive == "portions":
        return portion_steps(requests), longest
    return mixed_steps(requests)


@pytest.fixture(scope="module")
def replays(tmp_path_factory):
    """Every (model, dtype, drive) is replayed once per module and shared by the tests that look at it."""
    cache: dict = {}

    def get(model, dtype, drive):
        name, folder, requests, _ = model
        key = (name, dtype, drive)
        if key not in cache:
            steps, max_tokens = drive_steps(requests, drive)
            out = tmp_path_factory.mktemp(f"replay_{name}_{dtype}_{drive}")
            log = out / "pages.jsonl" if drive == "mixed" else None
            cache[key] = (steps, run_trace(folder, dtype, steps, out, max_tokens=max_tokens, pages_log=log), max_tokens, log)
        return cache[key]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
class TestReplay:
    def test_whole(self, model, dtype, replays):
        steps, results, _, _ = replays(model, dtype, "whole")
        compare_steps(steps, results, model[3], TOLERANCE[dtype])

    def test_last_32_one_by_one(self, model, dtype, replays):
        steps, results, _, _ = replays(model, dtype, "last32")
        compare_steps(steps, results, model[3], TOLERANCE[dtype])

    def test_portions_of_changing_size(self, model, dtype, replays):
        steps, results, _, _ = replays(model, dtype, "portions")
        assert min(len(e["tokens"]) for s in steps for e in s["entries"]) == 2
        compare_steps(steps, results, model[3], TOLERANCE[dtype])

    def test_mixed_with_page_reuse(self, model, dtype, replays):
        name, folder, requests, reference = model
        steps, results, peak, log = replays(model, dtype, "mixed")
        assert max(len(s["entries"]) for s in steps) == 4
        assert peak < sum(round64(len(ids)) for ids in requests.values())  # the pool cannot hold all: pages are reused
        compare_steps(steps, results, reference, TOLERANCE[dtype])
        # which pages: none in two tables at any time, given back only by their holder, and pages that one request gave
        # back were later another request's (the reference reads its pool back for the same reason: pages nobody owns are
        # unchanged, helios/crates/helios-hal/tests/batch_hw.rs:148-157)
        pool_pages = -(-max(64, round64(peak)) // 16)
        report = check_pages_log(log, steps, pool_pages)
        assert report["handed_on"] >= 4, report


def test_float32_logits_are_the_same_bits_however_the_requests_are_cut(model, replays):
    """Whole, with the last 32 tokens one by one, in portions down to two tokens, and mixed with other requests over
    reused pages: the float32 logits of the same (request, position) are the same bits in all four, not only close to
    the plain implementation (the reference holds a weaker form per bucket, helios/crates/helios-hal/tests/batch_hw.rs:122-163)."""
    rows = {drive: logits_by_position(*replays(model, "float32", drive)[:2]) for drive in DRIVES}
    whole = rows["whole"]
    assert len(whole) == sum(len(ids) for ids in model[2].values())
    for drive in DRIVES[1:]:
        assert rows[drive], drive
        for key, got in rows[drive].items():
            assert np.array_equal(got.view(np.uint32), whole[key].view(np.uint32)), f"{drive}: request {key[0]} position {key[1]} differs from the whole run"
    assert set(rows["portions"]) == set(whole) and set(rows["mixed"]) == set(whole)


def test_mixed_replay_with_every_product_on_the_tcgen05_kernel(model, tmp_path):
    """The same mixed trace in bfloat16 with HYPERION_B200_GEMM=own: every projection, large or small, goes through
    the package's tcgen05 kernel instead of the library."""
    name, folder, requests, reference = model
    steps, peak = mixed_steps(requests)
    results = run_trace(folder, "bfloat16", steps, tmp_path, max_tokens=peak, env={"HYPERION_B200_GEMM": "own"})
    compare_steps(steps, results, reference, TOLERANCE["bfloat16"])


@pytest.fixture(scope="module")
def model_c(tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("model_C"), "C")
    requests = requests_for("C")
    return "C", folder, requests, {rid: plain_logits(folder, ids) for rid, ids in requests.items()}


@pytest.mark.parametrize("page_size", [8, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_replay_with_other_page_sizes(model_c, replays, dtype, page_size, tmp_path):
    """The mixed trace (pages reused) on the configuration with heads of 64, with pages of 8 and of 64 tokens: the
    page size is a parameter of the cache and of every kernel that walks it, not a constant.  In float32 the logits are
    the bits of the whole run over pages of 16: where a key lies in the cache changes nothing."""
    _, folder, requests, reference = model_c
    steps, peak = mixed_steps(requests)
    results = run_trace(folder, dtype, steps, tmp_path, max_tokens=peak, page_size=page_size)
    compare_steps(steps, results, reference, TOLERANCE[dtype])
    if dtype == "float32":
        whole = logits_by_position(*replays(model_c, "float32", "whole")[:2])
        for key, got in logits_by_position(steps, results).items():
            assert np.array_equal(got.view(np.uint32), whole[key].view(np.uint32)), f"pages of {page_size}: request {key[0]} position {key[1]}"
