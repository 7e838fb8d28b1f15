"""The kernels and the engine at the sizes the benchmark runs, each against the plain implementation in float64:
attention alone at contexts of 2,048 to 4,096 (and of tens of thousands, with one key that dominates) with the 7B
configuration's 28/4 heads of 128 and pages of 16, and a two-layer model of the 7B configuration's widths under mixed
steps, decode batches of 8 and 64, and replayed graphs."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import TOLERANCE, compare_steps, random_ids, run_trace
from plain import qwen2_plain as plain
from test_kernels_gpu import DEV, rnd
from test_replay_gpu import mixed_steps

pytestmark = pytest.mark.gpu

HEADS, KV_HEADS, HEAD_DIM, PAGE = 28, 4, 128, 16
# Declared before the first run: bfloat16 queries, keys, values and probabilities (2^-9 relative each) through one softmax.
ATTENTION_TOLERANCE = 2 ** -7


def big_paged_case(contexts, seed, spare_pages=64):
    """Keys and values for requests of the given contexts on shuffled pages of one pool, on the device.  Slots nobody
    owns (the tails of last pages, pages outside every table) hold large finite values, as a reused page holds its last
    owner's keys and values: reading one of them moves the result by far more than the tolerance."""
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-c // PAGE) for c in contexts]
    pages = sum(blocks) + spare_pages
    order = torch.randperm(pages, generator=g).tolist()
    garbage = torch.where(torch.rand((pages, 2, KV_HEADS, PAGE, HEAD_DIM), generator=g) < 0.5, -1.0, 1.0) * 300.0
    cache = garbage.to(torch.bfloat16)
    table = torch.full((len(contexts), max(blocks) + 3), -1, dtype=torch.int32)
    keys, values = [], []
    for r, c in enumerate(contexts):
        k = rnd(c, KV_HEADS, HEAD_DIM, seed=seed * 100 + 2 * r, dtype=torch.bfloat16)
        v = rnd(c, KV_HEADS, HEAD_DIM, seed=seed * 100 + 2 * r + 1, dtype=torch.bfloat16)
        keys.append(k)
        values.append(v)
        for b in range(blocks[r]):
            page = order.pop()
            table[r, b] = page
            n = min(PAGE, c - b * PAGE)
            cache[page, 0, :, :n] = k[b * PAGE : b * PAGE + n].transpose(0, 1)
            cache[page, 1, :, :n] = v[b * PAGE : b * PAGE + n].transpose(0, 1)
    return cache.to(DEV), table.to(DEV), keys, values


def reference(q, keys, values, rows):
    """plain.attention in float64 on the device (the sizes are the benchmark's), per row (request, first position, count)."""
    outs, at = [], 0
    for request, first, count in rows:
        k, v = keys[request].to(DEV).double(), values[request].to(DEV).double()
        outs.append(plain.attention(q[at:at + count], k, v, torch.arange(first, first + count, device=DEV), torch.arange(k.shape[0], device=DEV),
                                    HEAD_DIM ** -0.5))
        at += count
    return torch.cat(outs)


@pytest.mark.parametrize("first", [0, 2048, 1029, 14336])
def test_prompt_attention_of_2048_tokens_at_the_benchmark_sizes(first):
    """One portion of 2,048 tokens from position 0, one from position 2,048 (context 4,096), one from an odd position
    (its context ends inside a page and inside a tile of keys) and one that ends at a context of 16,384 (every block
    walks some hundred tiles of keys, item after item) through the tile kernel the engine picks for heads of 128 and
    pages of 16."""
    from hyperion_b200.engine.batch import Row
    from hyperion_b200.ops import attention as fast
    from hyperion_b200.ops import raise_on_status

    count = 2048
    cache, table, keys, values = big_paged_case([first + count], seed=31 + first)
    q = rnd(count, (HEADS + 2 * KV_HEADS) * HEAD_DIM, seed=32, dtype=torch.bfloat16).to(DEV)
    size = fast.tile_rows(HEAD_DIM, PAGE)
    assert size == fast.TC_TILE_ROWS and fast.uses_tcgen05(HEAD_DIM, PAGE)
    tiles, items = fast.plan([Row(0, 0, count, first, 0)], fast.tile_tokens(HEADS, KV_HEADS, size))
    assert len(items) == 0
    token_row = torch.zeros(count, dtype=torch.int32, device=DEV)
    positions = torch.arange(first, first + count, dtype=torch.int32, device=DEV)
    out = torch.full((count, HEADS * HEAD_DIM), float("nan"), dtype=torch.bfloat16, device=DEV)
    fast.attention_tiles(q, HEADS, cache, table, token_row, positions, torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles) // 3,
                         HEAD_DIM ** -0.5, 0, out, tile_size=size)
    raise_on_status(torch.device(DEV))
    want = reference(q[:, : HEADS * HEAD_DIM].double().view(count, HEADS, HEAD_DIM), keys, values, [(0, first, count)])
    got = out.double().view(count, HEADS, HEAD_DIM)
    assert torch.isfinite(got).all()
    error = (got - want).abs().amax(dim=(1, 2)) / want.abs().max()
    assert error.max() <= ATTENTION_TOLERANCE, f"token {int(error.argmax())} (position {first + int(error.argmax())}): {float(error.max()):.3e}"


@pytest.mark.parametrize("batch", [1, 8, 64])
def test_decode_attention_at_contexts_of_2048_to_4096(batch):
    """Single tokens of `batch` requests whose contexts spread over 2,048 .. 4,096 through the split-key kernel: with the
    split count the engine fixes for a replayed graph (from the widest context its padded block tables can hold), with
    the count of a direct step, and with one split."""
    from hyperion_b200.ops import attention as fast
    from hyperion_b200.ops import raise_on_status

    contexts = [2048, 4096, 3072, 2049, 4095, 3000, 2500, 3584][:batch] if batch <= 8 else [2048 + (r * 2048) // 63 for r in range(64)]
    cache, table, keys, values = big_paged_case(contexts, seed=40 + batch)
    q = rnd(batch, (HEADS + 2 * KV_HEADS) * HEAD_DIM, seed=41, dtype=torch.bfloat16).to(DEV)
    token_row = torch.arange(batch, dtype=torch.int32, device=DEV)
    positions = torch.tensor([c - 1 for c in contexts], dtype=torch.int32, device=DEV)
    items = torch.arange(batch, dtype=torch.int32, device=DEV)
    rows = [(r, c - 1, 1) for r, c in enumerate(contexts)]
    want = reference(q[:, : HEADS * HEAD_DIM].double().view(batch, HEADS, HEAD_DIM), keys, values, rows)
    widest_pages = 64
    while widest_pages * PAGE < max(contexts):
        widest_pages *= 2  # a graphed step's table width: 64 pages times a power of two
    graph_splits = fast.choose_splits(batch, HEADS, KV_HEADS, widest_pages * PAGE)
    direct_splits = fast.choose_splits(batch, HEADS, KV_HEADS, max(contexts))
    for splits in sorted({1, graph_splits, direct_splits}):
        out = torch.full((batch, HEADS * HEAD_DIM), float("nan"), dtype=torch.bfloat16, device=DEV)
        fast.attention_tokens(q, HEADS, cache, table, token_row, positions, items, batch, splits, HEAD_DIM ** -0.5, 0, out)
        raise_on_status(torch.device(DEV))
        got = out.double().view(batch, HEADS, HEAD_DIM)
        assert torch.isfinite(got).all(), f"{splits} splits: not finite"
        error = (got - want).abs().amax(dim=(1, 2)) / want.abs().max()
        assert error.max() <= ATTENTION_TOLERANCE, f"{splits} splits, row {int(error.argmax())} (context {contexts[int(error.argmax())]}): {float(error.max()):.3e}"


def test_decode_attention_finds_one_key_in_contexts_of_tens_of_thousands():
    """Random keys average a lost tile away when there are tens of thousands of them: here one key per request dominates
    every query (at the start, in the middle, at the last position but one, at the edge of a split), so the output is
    that key's value, or the kernel has skipped it."""
    from hyperion_b200.ops import attention as fast
    from hyperion_b200.ops import raise_on_status

    contexts = [16384, 32768, 20000, 9001]
    batch = len(contexts)
    cache, table, keys, values = big_paged_case(contexts, seed=60)
    direction = rnd(HEAD_DIM, seed=61).to(torch.bfloat16)
    spots = [5, 32768 // 2 + 63, 20000 - 2, 9001 - 64 * 47]
    for r, spot in enumerate(spots):
        keys[r][spot] = direction * 4
        cache[table[r, spot // PAGE], 0, :, spot % PAGE] = (direction * 4).to(DEV)
    q = (direction.float() * 4).repeat(batch, HEADS + 2 * KV_HEADS).to(torch.bfloat16).to(DEV)
    token_row = torch.arange(batch, dtype=torch.int32, device=DEV)
    positions = torch.tensor([c - 1 for c in contexts], dtype=torch.int32, device=DEV)
    items = torch.arange(batch, dtype=torch.int32, device=DEV)
    rows = [(r, c - 1, 1) for r, c in enumerate(contexts)]
    want = reference(q[:, : HEADS * HEAD_DIM].double().view(batch, HEADS, HEAD_DIM), keys, values, rows)
    for splits in sorted({1, 7, fast.choose_splits(batch, HEADS, KV_HEADS, max(contexts)), 64}):
        out = torch.full((batch, HEADS * HEAD_DIM), float("nan"), dtype=torch.bfloat16, device=DEV)
        fast.attention_tokens(q, HEADS, cache, table, token_row, positions, items, batch, splits, HEAD_DIM ** -0.5, 0, out)
        raise_on_status(torch.device(DEV))
        got = out.double().view(batch, HEADS, HEAD_DIM)
        assert torch.isfinite(got).all(), f"{splits} splits: not finite"
        assert (got - want).abs().max() <= ATTENTION_TOLERANCE * want.abs().max(), f"{splits} splits"
        for r, spot in enumerate(spots):
            distance = (got[r, 0] - values[r][spot, 0].double().to(DEV)).abs().max()
            assert distance < 0.05, f"{splits} splits: request {r} did not find its key at {spot} ({float(distance):.3f})"


@pytest.mark.parametrize("spot", [3, 10000 + 127, 128 * 77, 19999])
def test_prompt_attention_finds_one_key_in_a_context_of_twenty_thousand(spot):
    """A prompt portion of 300 tokens behind 20,000 cached ones, one of which (near the start, at the last and at the
    first key of a 128-key tile, right before the portion) dominates every query."""
    from hyperion_b200.engine.batch import Row
    from hyperion_b200.ops import attention as fast
    from hyperion_b200.ops import raise_on_status

    first, count = 20000, 300
    cache, table, keys, values = big_paged_case([first + count], seed=70)
    direction = rnd(HEAD_DIM, seed=71).to(torch.bfloat16)
    keys[0][spot] = direction * 4
    cache[table[0, spot // PAGE], 0, :, spot % PAGE] = (direction * 4).to(DEV)
    q = (direction.float() * 4).repeat(count, HEADS + 2 * KV_HEADS).to(torch.bfloat16).to(DEV)
    size = fast.tile_rows(HEAD_DIM, PAGE)
    tiles, items = fast.plan([Row(0, 0, count, first, 0)], fast.tile_tokens(HEADS, KV_HEADS, size))
    assert len(items) == 0
    token_row = torch.zeros(count, dtype=torch.int32, device=DEV)
    positions = torch.arange(first, first + count, dtype=torch.int32, device=DEV)
    out = torch.full((count, HEADS * HEAD_DIM), float("nan"), dtype=torch.bfloat16, device=DEV)
    fast.attention_tiles(q, HEADS, cache, table, token_row, positions, torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles) // 3,
                         HEAD_DIM ** -0.5, 0, out, tile_size=size)
    raise_on_status(torch.device(DEV))
    want = reference(q[:, : HEADS * HEAD_DIM].double().view(count, HEADS, HEAD_DIM), keys, values, [(0, first, count)])
    got = out.double().view(count, HEADS, HEAD_DIM)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() <= ATTENTION_TOLERANCE * want.abs().max()
    distance = (got[:, 0] - values[0][spot, 0].double().to(DEV)).abs().max()
    assert distance < 0.05, f"the key at {spot} was not found ({float(distance):.3f})"


# ------------------------------------------------------------------------------------------------ a model of real widths
def wide_config(vocab=2003):
    from hyperion_b200.config import Qwen2Config

    return Qwen2Config(num_hidden_layers=2, hidden_size=3584, intermediate_size=18944, num_attention_heads=HEADS, num_key_value_heads=KV_HEADS,
                       head_dim=HEAD_DIM, vocab_size=vocab, max_position_embeddings=4096, rope_theta=1e6, rms_norm_eps=1e-6,
                       tie_word_embeddings=False)


@pytest.fixture(scope="module")
def wide_folder(tmp_path_factory):
    from hyperion_b200.weights import write_model_folder

    return write_model_folder(tmp_path_factory.mktemp("wide") / "two_layers", "Qwen2ForCausalLM", wide_config(), seed=9, std=0.02)


@pytest.fixture(scope="module")
def wide_plain(wide_folder):
    """ids -> the plain implementation's float64 logits, its weights widened once and kept on the device."""
    config, weights = plain.read_model_folder(wide_folder)
    wide = {name: tensor.to(device=DEV, dtype=torch.float64) for name, tensor in weights.items()}
    yield lambda ids: plain.forward(config, wide, list(ids), device=DEV).cpu().numpy()
    wide.clear()
    torch.cuda.empty_cache()


# float32 at these widths: reductions of up to 18,944 terms in float against float64 (declared as for the one-layer test of
# the engine tests); bfloat16 as for the tiny models.
WIDE_TOLERANCE = {"float32": 1e-4, "bfloat16": TOLERANCE["bfloat16"]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_trace_at_the_widths_of_the_7b_configuration(wide_folder, wide_plain, dtype, tmp_path):
    """Up to four live requests, prompt portions of some beside single tokens of others, pages reused, through
    bin/trace_run on a two-layer model with hidden 3,584, 28/4 heads of 128 and intermediate 18,944."""
    config = wide_config()
    requests = {f"r{i}": random_ids(300 + i, n, config.vocab_size) for i, n in enumerate([150, 60, 200, 90, 120, 70])}
    want = {rid: wide_plain(ids) for rid, ids in requests.items()}
    steps, peak = mixed_steps(requests)
    assert max(len(s["entries"]) for s in steps) == 4
    results = run_trace(wide_folder, dtype, steps, tmp_path, max_tokens=peak)
    compare_steps(steps, results, want, WIDE_TOLERANCE[dtype])


def test_decode_batches_of_8_and_64_and_replayed_graphs_at_real_widths(wide_folder, wide_plain):
    """64 requests with prompts of 17 .. 80 tokens on the bfloat16 engine: steps of 8 and of 64 single tokens (the swapped
    tcgen05 product with 16-, 32- and 64-row tiles at K = 18,944, its split-K pieces read by the norm, the library's
    products where the engine uses them), each three times so that the third is a replayed graph, and a prompt portion of
    one shape four times so that the last is a replay too; every row against the plain implementation."""
    from hyperion_b200.api import Engine
    from hyperion_b200.engine.batch import StepEntry

    config = wide_config()
    tolerance = WIDE_TOLERANCE["bfloat16"]
    engine = Engine.from_folder(wide_folder, dtype="bfloat16", page_size=16, max_tokens=64 * 128, max_requests=66)
    prompts = [random_ids(500 + i, 17 + i, config.vocab_size) for i in range(64)]
    tails = [random_ids(700 + i, 6, config.vocab_size) for i in range(64)]
    want = [wide_plain(prompts[i] + tails[i]) for i in range(64)]

    def check(logits, rows, what):
        got = logits.float().cpu().numpy()
        for r, (request, position) in enumerate(rows):
            ref = want[request][position]
            error = np.abs(got[r] - ref).max() / np.abs(ref).max()
            assert error <= tolerance, f"{what}: request {request} position {position}: {error:.3e}"

    for first in range(0, 64, 8):  # prompts, eight a step, the last position of each wanted
        batch = range(first, first + 8)
        logits = engine.step([StepEntry(i, prompts[i], [len(prompts[i]) - 1]) for i in batch])
        check(logits, [(i, len(prompts[i]) - 1) for i in batch], "prompts")
    fed = [0] * 64
    for size, members in ((8, list(range(8, 16))), (24, list(range(16, 40))), (64, list(range(64)))):
        for repeat in range(3):  # first sighting direct, second captured, third replayed
            logits = engine.step([StepEntry(i, [tails[i][fed[i]]], [0]) for i in members])
            check(logits, [(i, len(prompts[i]) + fed[i]) for i in members], f"decode batch {size}, step {repeat}")
            for i in members:
                fed[i] += 1
    assert engine.runner.graph_launches > 0
    replays_before = engine.runner.graph_launches
    portion = 128
    for k in range(4):  # the same shape four times: direct, direct, captured, replayed
        ids = random_ids(900 + k, portion, config.vocab_size)
        ref = wide_plain(ids)
        logits = engine.step([StepEntry(("portion", k), ids, [0, portion - 1])]).float().cpu().numpy()
        for r, position in enumerate((0, portion - 1)):
            error = np.abs(logits[r] - ref[position]).max() / np.abs(ref[position]).max()
            assert error <= tolerance, f"portion {k} position {position}: {error:.3e}"
        engine.finish(("portion", k))
    assert engine.runner.graph_launches > replays_before  # the fourth was a replay
    engine.check()
