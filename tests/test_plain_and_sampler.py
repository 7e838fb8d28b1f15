"""The plain implementation against the reference's committed oracle, its parts against direct
formulas, and the host sampling rule (no GPU)."""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from plain import qwen2_plain as plain

from hyperion_b200.sampling import InvalidParameter, SamplingParams, philox4x32_10, reference_sample, uniform

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_plain_implementation_meets_the_reference_oracle():
    """Float32 top-20 logits and logsumexp the reference published for its tiny checkpoint, at every
    teacher-forced position, within the tolerance the oracle file declares (0.02); the plain
    implementation actually agrees to about 1e-6."""
    config, weights = plain.read_model_folder(GOLDEN / "qwen2-tiny-sharded")
    oracle = json.loads((GOLDEN / "qwen2-tiny-oracle.json").read_text())
    worst = 0.0
    for prompt in oracle["prompts"]:
        logits = plain.forward(config, weights, prompt["ids"] + prompt["generated_ids"])
        for row in prompt["positions"]:
            mine = logits[row["position"]]
            worst = max(worst, max(abs(float(mine[i]) - v) for i, v in zip(row["top_ids"], row["top_logits"])))
            worst = max(worst, abs(float(torch.logsumexp(mine, 0)) - row["logsumexp"]))
            assert int(torch.argmax(mine)) == row["argmax"]
    assert worst <= 1e-5 < oracle["tolerance"]["max_abs_top_logits"]


def test_engine_reads_the_sharded_fixture_like_the_plain_reader():
    from hyperion_b200.models import read_model_config
    from hyperion_b200.weights import read_all

    architecture, config = read_model_config(GOLDEN / "qwen2-tiny-sharded")
    assert (config.num_hidden_layers, config.head_dim, config.rope_theta, config.eos_token_ids) == (2, 16, 10000.0, (127,))
    mine = read_all(GOLDEN / "qwen2-tiny-sharded")
    _, theirs = plain.read_model_folder(GOLDEN / "qwen2-tiny-sharded")
    assert set(mine) == set(theirs) and all(torch.equal(mine[n], theirs[n]) for n in mine)


def test_plain_parts_against_direct_formulas():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(plain.rmsnorm(x, torch.tensor([2.0, 0.5], dtype=torch.float64), 0.0), torch.tensor([[6 / math.sqrt(12.5), 2 / math.sqrt(12.5)]], dtype=torch.float64))
    cos, sin = plain.rope_tables(torch.tensor([0, 3]), 4, 100.0)
    assert torch.allclose(cos[1], torch.tensor([math.cos(3.0), math.cos(0.3)], dtype=torch.float64))
    rotated = plain.rope(torch.tensor([[[1.0, 2.0, 3.0, 4.0]]], dtype=torch.float64).repeat(2, 1, 1), cos, sin)
    assert torch.allclose(rotated[0], torch.tensor([[1.0, 2.0, 3.0, 4.0]], dtype=torch.float64))
    c, s = math.cos(3.0), math.sin(3.0)
    assert torch.allclose(rotated[1, 0, [0, 2]], torch.tensor([1 * c - 3 * s, 3 * c + 1 * s], dtype=torch.float64))
    # attention: one query over two keys, by hand; then the causal mask and the window
    q = torch.tensor([[[1.0, 0.0]]], dtype=torch.float64)
    k = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]]], dtype=torch.float64)
    v = torch.tensor([[[10.0, 0.0]], [[0.0, 10.0]]], dtype=torch.float64)
    out = plain.attention(q, k, v, torch.tensor([1]), torch.tensor([0, 1]), 1.0)
    w = math.e / (math.e + 1)
    assert torch.allclose(out[0, 0], torch.tensor([10 * w, 10 * (1 - w)], dtype=torch.float64))
    assert torch.allclose(plain.attention(q, k, v, torch.tensor([0]), torch.tensor([0, 1]), 1.0)[0, 0], v[0, 0])
    assert torch.allclose(plain.attention(q, k, v, torch.tensor([1]), torch.tensor([0, 1]), 1.0, window=1)[0, 0], v[1, 0])
    # grouped heads: heads 0,1 read kv head 0 and heads 2,3 read kv head 1
    q4 = torch.zeros(1, 4, 2, dtype=torch.float64)
    kv = torch.tensor([[[1.0, 1.0], [2.0, 2.0]]], dtype=torch.float64)
    assert plain.attention(q4, kv, kv, torch.tensor([0]), torch.tensor([0]), 1.0)[0, :, 0].tolist() == [1.0, 1.0, 2.0, 2.0]
    g = torch.tensor([[0.0, 1.0]], dtype=torch.float64)
    eye = torch.eye(2, dtype=torch.float64)
    assert torch.allclose(plain.swiglu_mlp(g, eye, eye, eye), torch.tensor([[0.0, 1 / (1 + math.exp(-1))]], dtype=torch.float64))


def test_philox_known_answers():
    # the known-answer vectors of Philox4x32-10 from the Random123 distribution
    assert philox4x32_10([0, 0, 0, 0], [0, 0]) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert philox4x32_10([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert philox4x32_10([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0]) == [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]
    assert 0.0 <= uniform(123, 0) < 1.0 and uniform(123, 0) != uniform(123, 1) and uniform(123, 5) == uniform(123, 5)


def test_sampling_params_ranges():
    for bad in (dict(temperature=2.5), dict(temperature=-0.1), dict(top_p=1.5), dict(top_k=-1), dict(repetition_penalty=0.0),
                dict(temperature=0.0, repetition_penalty=1.2), dict(max_tokens=0), dict(seed=-1)):
        with pytest.raises(InvalidParameter):
            SamplingParams(**bad).validated()
    assert SamplingParams().validated().seed is not None  # an absent seed is drawn
    assert SamplingParams(seed=7).validated().seed == 7


def test_reference_sampler_rule():
    logits = np.array([2.0, 1.0, 0.0, 3.0, -1.0], dtype=np.float32)
    assert reference_sample(logits, SamplingParams(temperature=0.0).validated(), 0)[0] == 3
    assert reference_sample(np.array([1.0, 5.0, 5.0, np.nan], dtype=np.float32), SamplingParams(temperature=0.0).validated(), 0)[0] == 1
    for step in range(50):
        token, info = reference_sample(logits, SamplingParams(temperature=1.0, top_k=2, seed=3).validated(), step)
        assert token in (0, 3) and sorted(info["kept"].tolist()) == [0, 3]
        token, info = reference_sample(logits, SamplingParams(temperature=1.0, top_p=0.6, seed=3).validated(), step)
        assert token == 3  # the largest token alone holds 0.64 of the mass
        token, info = reference_sample(logits, SamplingParams(temperature=1.0, top_p=0.7, seed=3).validated(), step)
        assert sorted(info["kept"].tolist()) == [0, 3]
    # the penalty divides positive and multiplies negative logits of generated tokens only
    penal = SamplingParams(temperature=1.0, top_k=1, repetition_penalty=4.0, seed=1).validated()
    assert reference_sample(logits, penal, 0, generated=[3])[0] == 0
    assert reference_sample(logits, penal, 0, generated=[])[0] == 3
    counts = np.zeros(5)
    sampling = SamplingParams(temperature=1.0, seed=11).validated()
    for step in range(4000):
        counts[reference_sample(logits, sampling, step)[0]] += 1
    expected = np.exp(logits) / np.exp(logits).sum() * 4000
    assert (((counts - expected) ** 2) / expected).sum() < 25
