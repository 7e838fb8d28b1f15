"""The engine on the GPU beyond replay: long decoding, the first tokens of a sequence, generation
through the Python entry point with greedy and temperature sampling, and what happens when pages
run out."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import STATED, TINY, TOLERANCE, make_folder, make_stated_folder, plain_logits, random_ids
from plain import qwen2_plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("engine_models")
    return {name: make_folder(root, name) for name in TINY}


def engine_for(folder, dtype, **options):
    from hyperion_b200.api import Engine

    options.setdefault("page_size", 16)
    options.setdefault("max_tokens", 2048)
    options.setdefault("max_requests", 8)
    return Engine.from_folder(folder, dtype=dtype, **options)


def relative_error(got: np.ndarray, want: np.ndarray) -> float:
    return float(np.abs(got - want).max() / np.abs(want).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_token_by_token(folders, name, dtype):
    from hyperion_b200.engine.batch import StepEntry

    config, seed = TINY[name]
    ids = random_ids(seed + 40, 330, config.vocab_size)
    want = plain_logits(folders[name], ids)
    engine = engine_for(folders[name], dtype, page_size=8 if name == "A" else 32, max_tokens=384)
    logits = engine.step([StepEntry("r", ids[:10], [9])])
    worst = relative_error(logits.cpu().numpy()[0], want[9])
    for k in range(10, len(ids)):
        logits = engine.step([StepEntry("r", [ids[k]], [0])])
        worst = max(worst, relative_error(logits.cpu().numpy()[0], want[k]))
    engine.check()
    assert worst <= TOLERANCE[dtype], worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(folders, dtype):
    from hyperion_b200.engine.batch import StepEntry

    config, seed = TINY["B"]
    ids = random_ids(77, 6, config.vocab_size)
    want = plain_logits(folders["B"], ids)
    engine = engine_for(folders["B"], dtype)
    for k, token in enumerate(ids):  # positions 0, 1, 2, ... one at a time: a one-token prompt, then decoding
        logits = engine.step([StepEntry("one", [token], [0])])
        assert relative_error(logits.cpu().numpy()[0], want[k]) <= TOLERANCE[dtype]
    single = engine.step([StepEntry("single", [ids[0]], [0])])  # a prompt of exactly one token
    assert relative_error(single.cpu().numpy()[0], want[0]) <= TOLERANCE[dtype]
    pair = engine.step([StepEntry("pair", ids[:2], [0, 1])])
    assert relative_error(pair.cpu().numpy(), want[:2]) <= TOLERANCE[dtype]


def test_float32_logits_are_bit_identical_however_the_work_is_cut(folders):
    from hyperion_b200.engine.batch import StepEntry

    config, _ = TINY["A"]
    ids = random_ids(5, 90, config.vocab_size)
    other = random_ids(6, 50, config.vocab_size)
    engine = engine_for(folders["A"], "float32", page_size=4)
    whole = engine.step([StepEntry("w", ids, list(range(90)))]).cpu()
    pieces = []
    at = 0
    engine.step([StepEntry("noise", other[:17], [])])
    for n in (3, 1, 40, 2, 44):
        out = engine.step([StepEntry("p", ids[at:at + n], list(range(n))), StepEntry("noise", other[17 + at // 4: 18 + at // 4], [0])])
        pieces.append(out.cpu()[:n])
        at += n
    assert torch.equal(torch.cat(pieces), whole)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_the_plain_implementation(folders, name):
    from hyperion_b200.sampling import SamplingParams

    config, seed = TINY[name]
    prompts = [random_ids(200 + i, n, config.vocab_size) for i, n in enumerate([5, 17, 31])]
    plain_config, weights = qwen2_plain.read_model_folder(folders[name])
    want = [qwen2_plain.greedy(plain_config, weights, prompt, 8) for prompt in prompts]
    engine = engine_for(folders[name], "float32")
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    assert got == want
    # bfloat16: teacher-forced on its own tokens, every choice must be the plain argmax or within the
    # bfloat16 tolerance of it (a near tie may flip)
    engine = engine_for(folders[name], "bfloat16")
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for prompt, tokens in zip(prompts, got):
        logits = plain_logits(folders[name], prompt + tokens)
        for i, token in enumerate(tokens):
            row = logits[len(prompt) + i - 1]
            assert row.max() - row[token] <= 2 * TOLERANCE["bfloat16"] * np.abs(row).max()


def test_temperature_sampling_follows_the_host_rule_under_chunked_mixed_steps(folders):
    """Four prompts of 1, 9, 40 and 63 tokens, prompt portions of at most 16 tokens mixed with
    decoding, 12 tokens each at temperature 0.8: every token the engine picked is the token the host
    rule picks from the plain implementation's logits, with the same seed and draw counter."""
    from hyperion_b200.sampling import SamplingParams, reference_sample

    config, _ = TINY["B"]
    prompts = [random_ids(300 + i, n, config.vocab_size) for i, n in enumerate([1, 9, 40, 63])]
    params = [SamplingParams(temperature=0.8, seed=1000 + i, max_tokens=12, ignore_eos=True) for i in range(4)]
    engine = engine_for(folders["B"], "float32")
    got = engine.generate(prompts, params, max_batch_tokens=16, prefill_chunk_busy=16)
    assert [len(g) for g in got] == [12] * 4
    for prompt, tokens, p in zip(prompts, got, params):
        logits = plain_logits(folders["B"], prompt + tokens)
        for i, token in enumerate(tokens):
            want, info = reference_sample(logits[len(prompt) + i - 1], p.validated(), i, tokens[:i])
            if want != token:
                kept = info["kept"].tolist()
                j = kept.index(token)
                assert (info["cdf"][j - 1] if j else 0.0) - 1e-5 <= info["u"] <= info["cdf"][j] + 1e-5
    # the same seeds give the same tokens whatever else is in the batch
    alone = engine.generate([prompts[2]], params[2])
    assert alone[0] == got[2]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_two_tiny_configurations_as_stated_run_their_stated_workloads(tmp_path, dtype):
    """The sizes, N(0, 0.02) weights and workloads the benchmark file gives its two tiny configurations: A (seed 0) three
    prompts of 5, 17 and 31 tokens and 8 greedy tokens each; B (seed 1) four prompts of 1, 9, 40 and 63 tokens in portions
    of 16 mixed with decoding, 12 tokens at temperature 0.8.  With weights this small the logits are nearly flat, so a
    greedy choice is held to the plain logits by distance (the plain argmax, or within the tolerance of it), and a sampled
    one to the host rule."""
    from hyperion_b200.sampling import SamplingParams, reference_sample

    tolerance = TOLERANCE[dtype]
    config, _ = STATED["A"]
    folder = make_stated_folder(tmp_path, "A")
    prompts = [random_ids(200 + i, n, config.vocab_size) for i, n in enumerate([5, 17, 31])]
    engine = engine_for(folder, dtype, max_tokens=256)
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for prompt, tokens in zip(prompts, got):
        assert len(tokens) == 8
        logits = plain_logits(folder, prompt + tokens)
        for i, token in enumerate(tokens):
            row = logits[len(prompt) + i - 1]
            assert row.max() - row[token] <= 2 * tolerance * np.abs(row).max()
    config, _ = STATED["B"]
    folder = make_stated_folder(tmp_path, "B")
    prompts = [random_ids(300 + i, n, config.vocab_size) for i, n in enumerate([1, 9, 40, 63])]
    params = [SamplingParams(temperature=0.8, seed=1000 + i, max_tokens=12, ignore_eos=True) for i in range(4)]
    engine = engine_for(folder, dtype, max_tokens=512)
    got = engine.generate(prompts, params, max_batch_tokens=16, prefill_chunk_busy=16)
    assert [len(g) for g in got] == [12] * 4
    slack = 1e-5 if dtype == "float32" else 0.05  # how far the draw may lie beyond the interval the plain logits give the token
    for prompt, tokens, p in zip(prompts, got, params):
        logits = plain_logits(folder, prompt + tokens)
        for i, token in enumerate(tokens):
            want, info = reference_sample(logits[len(prompt) + i - 1], p.validated(), i, tokens[:i])
            if want != token:
                kept = info["kept"].tolist()
                j = kept.index(token)
                assert (info["cdf"][j - 1] if j else 0.0) - slack <= info["u"] <= info["cdf"][j] + slack


def test_top_k_top_p_penalty_through_generate(folders):
    from hyperion_b200.sampling import SamplingParams

    config, _ = TINY["A"]
    prompt = random_ids(9, 12, config.vocab_size)
    engine = engine_for(folders["A"], "float32")
    params = SamplingParams(temperature=1.5, top_k=1, seed=5, max_tokens=6, ignore_eos=True)
    greedy = engine.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    assert engine.generate([prompt], params) == greedy  # top_k = 1 is the argmax whatever the temperature
    penalised = engine.generate([prompt], SamplingParams(temperature=1.0, top_k=1, repetition_penalty=50.0, seed=5, max_tokens=20, ignore_eos=True))[0]
    assert len(set(penalised)) >= 15  # a heavy penalty keeps generated tokens from coming back


def test_eos_stops_and_is_not_emitted(folders, tmp_path):
    import json
    import shutil

    from hyperion_b200.sampling import SamplingParams

    config, _ = TINY["A"]
    prompt = random_ids(10, 7, config.vocab_size)
    engine = engine_for(folders["A"], "float32")
    free_run = engine.generate([prompt], SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))[0]
    folder = tmp_path / "with_eos"
    shutil.copytree(folders["A"], folder)
    document = json.loads((folder / "config.json").read_text())
    document["eos_token_id"] = free_run[4]
    (folder / "config.json").write_text(json.dumps(document))
    engine = engine_for(folder, "float32")
    tokens, reasons = engine.generate([prompt], SamplingParams(temperature=0.0, max_tokens=10), return_reasons=True)
    first = free_run.index(free_run[4])
    assert tokens[0] == free_run[:first] and reasons == ["stop"]


def test_running_ahead_of_the_host_changes_nothing(folders, tmp_path):
    """Six requests, two of which meet an end-of-sequence token, greedy and at temperature 0.9, in a pool
    so small that requests wait: with the next step launched before the last ids reach the host, tokens
    and reasons are those of the step-by-step loop, and every page comes back."""
    import json
    import shutil

    from hyperion_b200.sampling import SamplingParams

    config, _ = TINY["A"]
    prompts = [random_ids(500 + i, n, config.vocab_size) for i, n in enumerate([5, 33, 18, 47, 2, 26])]
    params = [SamplingParams(temperature=0.0 if i % 2 else 0.9, seed=70 + i, max_tokens=4 + 3 * i, ignore_eos=True) for i in range(6)]
    free_run = engine_for(folders["A"], "float32").generate(prompts, params, lookahead=False)
    folder = tmp_path / "with_eos"
    shutil.copytree(folders["A"], folder)
    document = json.loads((folder / "config.json").read_text())
    document["eos_token_id"] = [free_run[3][5], free_run[5][2]]
    (folder / "config.json").write_text(json.dumps(document))
    params = [SamplingParams(temperature=p.temperature, seed=p.seed, max_tokens=p.max_tokens) for p in params]
    results = []
    for lookahead in (False, True):
        engine = engine_for(folder, "float32", max_tokens=160, max_requests=3)  # 10 pages
        seen = []
        results.append(engine.generate(prompts, params, max_batch_tokens=24, prefill_chunk_busy=8, return_reasons=True, lookahead=lookahead,
                                       on_token=lambda index, token: seen.append((index, token))))
        assert sorted(seen) == sorted((i, t) for i, tokens in enumerate(results[-1][0]) for t in tokens)
        engine.cache.check()
        assert engine.cache.free_pages() == 10 and not engine.cache.live_requests
    assert results[0] == results[1]
    assert "stop" in results[0][1] and "length" in results[0][1]


def test_small_pool_makes_requests_wait_and_a_hopeless_one_fail(folders):
    from hyperion_b200.sampling import SamplingParams

    config, _ = TINY["A"]
    prompts = [random_ids(400 + i, n, config.vocab_size) for i, n in enumerate([30, 50, 20, 45, 300, 25])]
    params = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    roomy = engine_for(folders["A"], "float32", max_tokens=4096)
    want = roomy.generate(prompts, params)
    tight = engine_for(folders["A"], "float32", page_size=16, max_tokens=128, max_requests=4)  # 8 pages
    got, reasons = tight.generate(prompts, params, return_reasons=True)
    assert reasons[4].startswith("needs 20 pages") and got[4] == []
    for i in (0, 1, 2, 3, 5):
        assert got[i] == want[i] and reasons[i] == "length"
    tight.cache.check()
    assert tight.cache.free_pages() == 8 and not tight.cache.live_requests


def test_a_bad_step_is_refused_whole(folders):
    from hyperion_b200.cache import OutOfPages
    from hyperion_b200.engine.batch import BadStep, StepEntry

    config, _ = TINY["A"]
    engine = engine_for(folders["A"], "float32", max_tokens=64)
    engine.step([StepEntry("a", [1, 2, 3], [])])
    for bad in ([StepEntry("a", [4], [0]), StepEntry("a", [5], [0])], [StepEntry("b", [], [])], [StepEntry("b", [config.vocab_size], [])],
                [StepEntry("b", [1], [1])], []):
        with pytest.raises(BadStep):
            engine.step(bad)
    with pytest.raises(OutOfPages):
        engine.step([StepEntry("a", [7], [0]), StepEntry("c", list(range(100)), [])])
    assert engine.cache.length("a") == 3 and not engine.cache.has("b") and not engine.cache.has("c")
    engine.cache.check()
    out = engine.step([StepEntry("a", [7], [0])])
    assert out.shape == (1, config.vocab_size)


def test_real_layer_widths_against_the_plain_implementation(tmp_path):
    """One layer with the widths of the 7B configuration (hidden 3584, 28/4 heads of 128, intermediate 18944,
    vocabulary 152064, tied head): a 70-token prompt in two portions and four decoded tokens, float32 and
    bfloat16, against the plain float64 implementation.  Tolerances declared beforehand: float32 1e-4 of
    the largest logit (reductions of up to 18944 terms), bfloat16 as for the tiny models."""
    from hyperion_b200.api import Engine
    from hyperion_b200.config import Qwen2Config
    from hyperion_b200.engine.batch import StepEntry
    from hyperion_b200.weights import write_model_folder

    config = Qwen2Config(num_hidden_layers=1, hidden_size=3584, intermediate_size=18944, num_attention_heads=28, num_key_value_heads=4,
                         head_dim=128, vocab_size=152064, max_position_embeddings=4096, rope_theta=1e6, rms_norm_eps=1e-6,
                         tie_word_embeddings=True)
    folder = write_model_folder(tmp_path / "wide", "Qwen2ForCausalLM", config, seed=5, std=0.02)
    ids = random_ids(55, 74, config.vocab_size)
    want = plain_logits(folder, ids)
    for dtype, tolerance in (("float32", 1e-4), ("bfloat16", TOLERANCE["bfloat16"])):
        engine = Engine.from_folder(folder, dtype=dtype, page_size=16, max_tokens=256, max_requests=2)
        got = [engine.step([StepEntry("r", ids[:47], [0, 46])]).cpu().numpy(), engine.step([StepEntry("r", ids[47:70], [22])]).cpu().numpy()]
        assert relative_error(got[0], want[[0, 46]]) <= tolerance
        assert relative_error(got[1], want[[69]]) <= tolerance
        for k in range(70, 74):
            logits = engine.step([StepEntry("r", [ids[k]], [0])]).cpu().numpy()
            assert relative_error(logits, want[[k]]) <= tolerance, (dtype, k)
        engine.check()
        del engine
        torch.cuda.empty_cache()


@pytest.mark.parametrize("name", ["A", "C"])
def test_bfloat16_steps_give_the_same_bits_every_time(folders, name):
    """The same mixed steps (prompt portions, decoded tokens, graph replays among them) eight times over on one engine,
    with freed memory overwritten by NaN in between: a race or a read of memory nobody wrote shows as logits that
    change from run to run."""
    from hyperion_b200.engine.batch import StepEntry

    config, _ = TINY[name]
    engine = engine_for(folders[name], "bfloat16", max_tokens=1024, max_requests=4)
    prompts = [random_ids(600 + i, n, config.vocab_size) for i, n in enumerate([70, 33, 5])]

    def run(tag):
        logits = []  # copied at once: a replayed graph writes its output in place
        names = [f"{tag}{i}" for i in range(3)]
        logits.append(engine.step([StepEntry(names[0], prompts[0][:40], [0, 39]), StepEntry(names[1], prompts[1], [32])]).cpu())
        logits.append(engine.step([StepEntry(names[0], prompts[0][40:], [29]), StepEntry(names[2], prompts[2], [4]),
                                   StepEntry(names[1], [7], [0])]).cpu())
        for k in range(6):  # decoded tokens
            logits.append(engine.step([StepEntry(n, [11 + k], [0]) for n in names]).cpu())
        for n in names:
            engine.finish(n)
        return logits

    for warm in range(3):
        run(f"warm{warm}")  # from here on every step of these shapes is a replay (the library's products may round
    first = run("a")  # differently inside a captured graph than in a direct launch, so like is compared with like)
    # the bits that repeat are the right ones: every replayed step against the plain implementation
    tail = [11 + k for k in range(6)]
    want = [plain_logits(folders[name], ids) for ids in (prompts[0] + tail, prompts[1] + [7] + tail, prompts[2] + tail)]
    rows = [[(0, 0), (0, 39), (1, 32)], [(0, 69), (2, 4), (1, 33)]] + [[(0, 70 + k), (1, 34 + k), (2, 5 + k)] for k in range(6)]
    for step, (logits, places) in enumerate(zip(first, rows)):
        for r, (request, position) in enumerate(places):
            assert relative_error(logits[r].float().numpy(), want[request][position]) <= TOLERANCE["bfloat16"], (step, request, position)
    for repeat in range(8):
        poison = [torch.full((n,), float("nan"), device="cuda") for n in (1 << 12, 1 << 16, 1 << 20, 1 << 22)]
        del poison
        again = run(f"b{repeat}_")
        for step, (x, y) in enumerate(zip(first, again)):
            assert torch.equal(x, y), f"repeat {repeat}, step {step}: logits changed"
    engine.check()


def test_a_cache_that_cannot_fit_is_refused_with_the_numbers(folders):
    with pytest.raises(MemoryError, match=r"needs .* GiB .* are free"):
        engine_for(folders["A"], "bfloat16", max_tokens=10 ** 12)


def test_forty_requests_through_a_small_pool_running_ahead_or_not(folders, tmp_path):
    """Forty requests of random lengths and budgets, a tenth of the vocabulary as end-of-sequence tokens, a pool of 24
    pages and at most 5 live requests: the loop that runs ahead gives the tokens and reasons of the step-by-step loop,
    and every page and slot comes back."""
    import json
    import random
    import shutil

    from hyperion_b200.sampling import SamplingParams

    config, _ = TINY["B"]
    rng = random.Random(11)
    folder = tmp_path / "many_eos"
    shutil.copytree(folders["B"], folder)
    document = json.loads((folder / "config.json").read_text())
    document["eos_token_id"] = rng.sample(range(config.vocab_size), config.vocab_size // 10)
    (folder / "config.json").write_text(json.dumps(document))
    prompts = [random_ids(700 + i, rng.randrange(1, 60), config.vocab_size) for i in range(40)]
    params = [SamplingParams(temperature=rng.choice([0.0, 0.7, 1.3]), top_k=rng.choice([0, 5]), seed=900 + i, max_tokens=rng.randrange(1, 30))
              for i in range(40)]
    results = []
    for lookahead in (False, True):
        engine = engine_for(folder, "float32", page_size=16, max_tokens=24 * 16, max_requests=5)
        results.append(engine.generate(prompts, params, max_batch_tokens=48, prefill_chunk_busy=16, return_reasons=True, lookahead=lookahead))
        engine.cache.check()
        assert engine.cache.free_pages() == 24 and not engine.cache.live_requests
    assert results[0] == results[1]
    reasons = results[0][1]
    assert reasons.count("stop") >= 5 and reasons.count("length") >= 5


@pytest.mark.parametrize("lookahead", [False, True])
def test_a_callback_that_returns_false_cancels_its_request(folders, lookahead):
    from hyperion_b200.sampling import SamplingParams

    config, _ = TINY["A"]
    prompts = [random_ids(800 + i, 9 + i, config.vocab_size) for i in range(3)]
    params = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    engine = engine_for(folders["A"], "float32", max_tokens=256, max_requests=4)
    whole = engine.generate(prompts, params, lookahead=lookahead)
    got, reasons = engine.generate(prompts, params, return_reasons=True, lookahead=lookahead,
                                   on_token=lambda index, token: not (index == 1 and token == whole[1][4]))
    stop = whole[1].index(whole[1][4]) + 1  # the token the callback refused was still delivered
    assert got[1] == whole[1][:stop] and reasons[1] == "cancelled"
    assert got[0] == whole[0] and got[2] == whole[2] and reasons[0] == reasons[2] == "length"
    engine.cache.check()
    assert not engine.cache.live_requests


def test_random_traffic_through_the_bfloat16_kernels_leaves_nothing_behind():
    """Rounds of random requests (prompts up to 1,500 tokens beside decoding requests, random budgets, portion sizes and
    sampling) through a model wide enough for the tensor-core attention and products: no kernel reports anything, every
    page and slot comes back, and every request ends within its budget. The kernels' hand-overs between warps are
    timing-dependent; a traffic mix is what moves the timing."""
    import random

    from hyperion_b200.api import Engine
    from hyperion_b200.config import Qwen2Config
    from hyperion_b200.sampling import SamplingParams

    config = Qwen2Config(num_hidden_layers=2, hidden_size=1024, intermediate_size=2816, num_attention_heads=8, num_key_value_heads=2,
                         head_dim=128, vocab_size=3001, max_position_embeddings=4096, rope_theta=1e4, rms_norm_eps=1e-6,
                         tie_word_embeddings=False, eos_token_ids=tuple(range(0, 3001, 53)))
    engine = Engine.from_random("Qwen2ForCausalLM", config, seed=3, dtype="bfloat16", page_size=16, max_tokens=12000, max_requests=12)
    rng = random.Random(2)
    for _ in range(10):
        count = rng.randrange(3, 16)
        prompts = [random_ids(rng.randrange(10 ** 6), rng.randrange(1, 1500), config.vocab_size) for _ in range(count)]
        params = [SamplingParams(temperature=rng.choice([0.0, 0.8, 1.2]), top_k=rng.choice([0, 20]), top_p=rng.choice([1.0, 0.9]),
                                 seed=rng.randrange(10 ** 6), max_tokens=rng.randrange(1, 60)) for _ in range(count)]
        tokens, reasons = engine.generate(prompts, params, max_batch_tokens=rng.choice([512, 2048, 8192]),
                                          prefill_chunk_busy=rng.choice([64, 512, 2048]), return_reasons=True,
                                          lookahead=rng.random() < 0.8)
        engine.check()
        engine.cache.check()
        assert not engine.cache.live_requests and engine.cache.free_pages() == engine.cache.num_pages
        for made, reason, wanted in zip(tokens, reasons, params):
            assert reason in ("stop", "length")
            assert len(made) <= wanted.max_tokens and all(0 <= t < config.vocab_size for t in made)
            assert reason == "stop" or len(made) == wanted.max_tokens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_whose_offsets_pass_two_to_the_31_elements(dtype, tmp_path):
    """A pool of 2.3 million tokens per layer (2.4 G elements) with all but its last 400 pages held by another request:
    the request lives on pages whose element offsets do not fit 32 bits, and its logits (two prompt portions, then
    single tokens) are the bits it gets on the first pages of a small pool."""
    from hyperion_b200.api import Engine
    from hyperion_b200.config import Qwen2Config
    from hyperion_b200.engine.batch import StepEntry

    config = Qwen2Config(num_hidden_layers=1, hidden_size=1024, intermediate_size=1536, num_attention_heads=8, num_key_value_heads=4,
                         head_dim=128, vocab_size=2000, max_position_embeddings=4096, rope_theta=1e4, rms_norm_eps=1e-6,
                         tie_word_embeddings=True, eos_token_ids=(0,))
    ids = random_ids(5, 1500, config.vocab_size)
    later = random_ids(6, 6, config.vocab_size)

    def run(engine, held_pages):
        if held_pages:
            engine.cache.add_request("holder")
            engine.cache.extend("holder", held_pages * 16)
        rows = [engine.step([StepEntry("a", ids[:600], [599])]).float().cpu(),
                engine.step([StepEntry("a", ids[600:], [len(ids) - 601])]).float().cpu()]
        rows += [engine.step([StepEntry("a", [token], [0])]).float().cpu() for token in later]
        engine.check()
        return torch.cat(rows), engine.cache.table(0, "a")

    small = Engine.from_random("Qwen2ForCausalLM", config, seed=0, dtype=dtype, page_size=16, max_tokens=4096, max_requests=4)
    want, low = run(small, 0)
    del small
    torch.cuda.empty_cache()
    pages = 2_300_000 // 16
    big = Engine.from_random("Qwen2ForCausalLM", config, seed=0, dtype=dtype, page_size=16, max_tokens=pages * 16, max_requests=4)
    got, high = run(big, pages - 400)
    assert low[0] == 0 and high[0] == pages - 400 and high[0] * 16 * 2 * 4 * 128 > 2 ** 31
    assert torch.isfinite(got).all() and torch.equal(got, want)
    # and those bits are right: the same model as a folder (the seed gives the same weights) through the plain implementation
    from hyperion_b200.weights import write_model_folder

    folder = write_model_folder(tmp_path / "offsets", "Qwen2ForCausalLM", config, seed=0)
    reference = plain_logits(folder, ids + later, device="cuda")
    places = [599, len(ids) - 1] + [len(ids) + k for k in range(len(later))]
    tolerance = 1e-4 if dtype == "float32" else TOLERANCE["bfloat16"]
    for row, position in enumerate(places):
        assert relative_error(got[row].numpy(), reference[position]) <= tolerance, position


# ------------------------------------------------------------------------------------------------ anchors
GOLDEN = __import__("pathlib").Path(__file__).resolve().parent / "golden"


def bf16_step(x: float) -> float:
    """One bfloat16 step at the magnitude of x (helios/crates/helios-hal/src/oracle.rs:179-184)."""
    return 0.0 if x == 0.0 or not np.isfinite(x) else 2.0 ** (int(np.floor(np.log2(abs(x)))) - 7)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "decode"])
def test_the_engine_meets_the_reference_oracle_on_its_own_checkpoint(dtype, cutting):
    """The reference's committed tiny checkpoint (five shards, read by tensor name) through the engine, teacher-forced on
    the oracle's prompts and generated ids: at every recorded position the top-20 logits and the logsumexp are within the
    tolerance the oracle declares for a bfloat16 forward (0.02; float32 must be within 1e-5, like the plain implementation),
    and the argmax is the oracle's or a token of its tie group, whose width is the rule of
    helios/crates/helios-hal/src/oracle.rs:197-217: min(tolerance, max(the reference's own bfloat16 deviation at this
    position, two bfloat16 steps of the best logit)).  `decode`: the prompt in one step, then token by token."""
    import json

    from hyperion_b200.engine.batch import StepEntry

    oracle = json.loads((GOLDEN / "qwen2-tiny-oracle.json").read_text())
    declared = oracle["tolerance"]["max_abs_top_logits"]
    limit = 1e-5 if dtype == "float32" else declared
    assert oracle["bf16_vs_fp32"]["top_logits"] * 1.5 <= declared  # the oracle's tolerance is its bfloat16 drift times a margin, floored
    engine = engine_for(GOLDEN / "qwen2-tiny-sharded", dtype, max_tokens=1024, max_requests=4)
    worst = 0.0
    for index, prompt in enumerate(oracle["prompts"]):
        ids = prompt["ids"] + prompt["generated_ids"]
        places = [row["position"] for row in prompt["positions"]]
        if cutting == "whole":
            logits = engine.step([StepEntry(index, ids, places)]).float().cpu().numpy()
        else:
            head = len(prompt["ids"])
            parts = [engine.step([StepEntry(index, ids[:head], [head - 1])]).float().cpu().numpy()]
            for k in range(head, len(ids)):
                parts.append(engine.step([StepEntry(index, [ids[k]], [0])]).float().cpu().numpy())
            by_position = dict(zip(range(head - 1, len(ids)), (p[0] for p in parts)))
            logits = np.stack([by_position[p] for p in places])
        engine.finish(index)
        for row, record, deviation in zip(logits, prompt["positions"], prompt["bf16_deviation"]):
            top = max(abs(float(row[i]) - v) for i, v in zip(record["top_ids"], record["top_logits"]))
            peak = float(row.max())
            lse = peak + float(np.log(np.exp(row.astype(np.float64) - peak).sum()))
            worst = max(worst, top, abs(lse - record["logsumexp"]))
            picked = int(row.argmax())
            best = record["top_logits"][0]
            threshold = min(declared, max(deviation, 2 * bf16_step(best)))
            gap = best - record["top_logits"][record["top_ids"].index(picked)] if picked in record["top_ids"] else None
            assert picked == record["argmax"] or (gap is not None and gap <= threshold), (index, record["position"], picked, gap, threshold)
    assert worst <= limit, worst
    engine.check()


def test_random_weights_in_memory_and_as_a_folder_are_the_same_bits(tmp_path):
    """One generator for both forms: `Engine.from_random(seed)` (a kernel fills the tensors on the device) and
    `write_model_folder(seed)` made on the host (numpy) give equal tensors, whatever their sizes and names."""
    from hyperion_b200.api import Engine
    from hyperion_b200.models import DecoderModel, get_architecture
    from hyperion_b200.weights import random_tensors, read_all, write_model_folder
    from hyperion_b200.weights.random_init import random_tensor
    from hyperion_b200.parts.base import WeightSpec

    config, seed = TINY["B"]
    folder = write_model_folder(tmp_path / "host", "Qwen2ForCausalLM", config, seed, 0.06, device="cpu")
    stored = read_all(folder)
    entry = get_architecture("Qwen2ForCausalLM")
    model = DecoderModel(entry.build_spec(config), torch.bfloat16, torch.device("cuda"))
    made = random_tensors(model, seed, 0.06)
    assert set(made) == set(stored)
    for name, tensor in made.items():
        assert tensor.is_cuda and torch.equal(tensor.cpu().view(torch.int16), stored[name].view(torch.int16)), name
    norm = stored["model.norm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.02 and 0.04 < float(norm.std()) < 0.08
    # odd lengths, float32 storage, another seed and name: equal again, and different from the first
    for shape, dtype in (((7, 13), torch.float32), ((1,), torch.bfloat16), ((333,), torch.float32)):
        wanted = WeightSpec(shape)
        host, device = (random_tensor("x.weight", wanted, 5, 0.5, torch.device(d), dtype) for d in ("cpu", "cuda"))
        assert torch.equal(host, device.cpu())
    assert not torch.equal(random_tensor("x.weight", WeightSpec((333,)), 5, 0.5, torch.device("cuda"), torch.float32),
                           random_tensor("y.weight", WeightSpec((333,)), 5, 0.5, torch.device("cuda"), torch.float32))
    # the engine made from the seed steps like the engine loaded from the folder: bit for bit
    from hyperion_b200.engine.batch import StepEntry

    ids = random_ids(3, 40, config.vocab_size)
    a = Engine.from_random("Qwen2ForCausalLM", config, seed=seed, std=0.06, dtype="float32", max_tokens=128, max_requests=2)
    b = Engine.from_folder(folder, dtype="float32", max_tokens=128, max_requests=2)
    assert torch.equal(a.step([StepEntry("r", ids, [39])]), b.step([StepEntry("r", ids, [39])]))


def test_a_step_that_fails_at_launch_under_lookahead_leaves_the_others_their_tokens(folders):
    """A caller's own request holds pages the scheduler counts as free, so a step of the generation loop runs out of pages
    when it is launched: its requests fail and are released.  Three requests decode under a budget of two tokens a step,
    so they take turns and the one that was not in the failed step has a row in flight at that moment; it goes on and
    reports exactly the tokens it generates alone.  (The step after a failed one must not take the staging slot of the
    step still in flight.)"""
    from hyperion_b200.engine.batch import StepEntry
    from hyperion_b200.sampling import SamplingParams

    config, _ = TINY["A"]
    prompts = [random_ids(40 + i, 4, config.vocab_size) for i in range(3)]
    params = SamplingParams(temperature=0.0, max_tokens=36, ignore_eos=True)
    clean = engine_for(folders["A"], "float32", page_size=16, max_tokens=160, max_requests=4).generate(prompts, params)
    results = []
    for lookahead in (False, True):
        engine = engine_for(folders["A"], "float32", page_size=16, max_tokens=160, max_requests=4)  # 10 pages
        engine.step([StepEntry("held by the caller", random_ids(1, 60, config.vocab_size), [])])  # 4 of them; 9 are reserved
        results.append(engine.generate(prompts, params, max_batch_tokens=2, prefill_chunk_busy=2, return_reasons=True, lookahead=lookahead))
        engine.finish("held by the caller")
        engine.cache.check()
        assert not engine.cache.live_requests and engine.cache.free_pages() == 10
    (tokens, reasons), (tokens_ahead, reasons_ahead) = results
    assert sorted("OutOfPages" in r for r in reasons) == [False, True, True], reasons  # one step failed: its two requests
    assert reasons_ahead == reasons
    survivor = reasons.index("length")
    assert tokens[survivor] == clean[survivor] and tokens_ahead[survivor] == clean[survivor]
