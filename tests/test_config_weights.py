"""Configuration reading, the architecture registry, safetensors reading and weight errors (no GPU)."""
from __future__ import annotations

import json
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B

from hyperion_b200.config import ConfigError, Qwen2Config, read_generation_defaults
from hyperion_b200.models import DecoderModel, architecture_of, get_architecture, read_model_config
from hyperion_b200.weights import SafetensorsError, WeightsError, check_tensors, read_all, read_header, read_model_index, write_file, write_model_folder

QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "hidden_act": "silu", "hidden_size": 3584, "intermediate_size": 18944,
    "max_position_embeddings": 32768, "max_window_layers": 28, "model_type": "qwen2", "num_attention_heads": 28,
    "num_hidden_layers": 28, "num_key_value_heads": 4, "rms_norm_eps": 1e-06, "rope_theta": 1000000.0, "sliding_window": 131072,
    "tie_word_embeddings": False, "use_sliding_window": False, "vocab_size": 152064, "eos_token_id": 151645,
}


def test_reads_the_7b_config_with_defaults():
    config = Qwen2Config.from_hf_dict(QWEN25_7B)
    assert (config.num_hidden_layers, config.hidden_size, config.head_dim, config.num_key_value_heads) == (28, 3584, 128, 4)
    assert config.rope_theta == 1e6 and config.rms_norm_eps == 1e-6 and not config.tie_word_embeddings
    assert config.eos_token_ids == (151645,)
    assert config.attention_scale == pytest.approx(128 ** -0.5)


def test_round_trip_through_config_json():
    for config in (TINY_A, TINY_B):
        assert Qwen2Config.from_hf_dict(config.to_hf_dict()) == config


def test_rope_theta_from_rope_parameters():
    document = {k: v for k, v in QWEN25_7B.items() if k != "rope_theta"}
    document["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    assert Qwen2Config.from_hf_dict(document).rope_theta == 12345.0
    document["rope_parameters"]["rope_type"] = "yarn"
    with pytest.raises(ConfigError) as error:
        Qwen2Config.from_hf_dict(document)
    assert "rope_type" in str(error.value)


@pytest.mark.parametrize("change, key", [
    ({"rms_norm_eps": None}, "rms_norm_eps"), ({"tie_word_embeddings": None}, "tie_word_embeddings"),
    ({"rope_scaling": {"type": "linear", "factor": 2}}, "rope_scaling"), ({"use_sliding_window": True}, "use_sliding_window"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"partial_rotary_factor": 0.5}, "partial_rotary_factor"),
    ({"num_key_value_heads": 5}, "num_key_value_heads"), ({"vocab_size": 0}, "vocab_size"), ({"num_hidden_layers": True}, "num_hidden_layers"),
    ({"architectures": ["LlamaForCausalLM"]}, "architectures"), ({"query_pre_attn_scalar": 64}, "query_pre_attn_scalar"),
    ({"rope_theta": -1}, "rope_theta"),
])
def test_refusals_name_the_key(change, key):
    document = dict(QWEN25_7B)
    document.update(change)
    document = {k: v for k, v in document.items() if v is not None}
    with pytest.raises(ConfigError) as error:
        Qwen2Config.from_hf_dict(document)
    assert error.value.key == key


def test_registry_picks_the_model_by_architecture_name(tmp_path):
    assert architecture_of(QWEN25_7B).name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError):
        architecture_of({"architectures": ["NoSuchModel"]})
    with pytest.raises(KeyError):
        get_architecture("NoSuchModel")
    folder = write_model_folder(tmp_path / "m", "Qwen2ForCausalLM", TINY_A, seed=0)
    architecture, config = read_model_config(folder)
    assert config == TINY_A
    spec = architecture.build_spec(config)
    assert len(spec.layers) == 2 and [run.layer for run in spec.schedule] == [0, 1]
    assert spec.layers[0].mixer.params["heads"] == 4 and spec.layers[1].feed_forward.params["intermediate_size"] == 176


def test_generation_defaults_merge_eos_ids(tmp_path):
    folder = tmp_path / "g"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps({**QWEN25_7B, "eos_token_id": 7}))
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": [7, 9], "temperature": 0.7, "top_k": 20, "top_p": 0.8,
                                                                 "repetition_penalty": 1.05}))
    defaults = read_generation_defaults(folder)
    assert defaults.eos_token_ids == (7, 9) and defaults.temperature == 0.7 and defaults.top_k == 20
    (folder / "generation_config.json").write_text(json.dumps({"temperature": -1}))
    with pytest.raises(ConfigError):
        read_generation_defaults(folder)


def test_random_folder_has_every_tensor_in_bfloat16(tmp_path):
    folder = write_model_folder(tmp_path / "b", "Qwen2ForCausalLM", TINY_B, seed=1)
    tensors = read_all(folder)
    assert "lm_head.weight" in tensors and tensors["lm_head.weight"].shape == (523, 192)
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    assert tensors["model.layers.2.self_attn.k_proj.bias"].shape == (32,)
    norm = tensors["model.norm.weight"].float()
    assert abs(norm.mean() - 1.0) < 0.02 and norm.std() > 0.005  # 1 + N(0, 0.02)
    again = read_all(write_model_folder(tmp_path / "b2", "Qwen2ForCausalLM", TINY_B, seed=1))
    assert all(torch.equal(tensors[n], again[n]) for n in tensors)
    other = read_all(write_model_folder(tmp_path / "b3", "Qwen2ForCausalLM", TINY_B, seed=2))
    assert not torch.equal(tensors["lm_head.weight"], other["lm_head.weight"])
    tied = read_all(write_model_folder(tmp_path / "a", "Qwen2ForCausalLM", TINY_A, seed=0))
    assert "lm_head.weight" not in tied


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_model_folder(tmp_path / "m", "Qwen2ForCausalLM", TINY_A, seed=0)
    tensors = read_all(folder)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(16, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 65, dtype=torch.bfloat16)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    (folder / "model.safetensors").unlink()
    write_file(folder / "model.safetensors", tensors)
    architecture, config = read_model_config(folder)
    model = DecoderModel(architecture.build_spec(config), torch.float32, torch.device("meta"))
    with pytest.raises(WeightsError) as error:
        check_tensors(read_model_index(folder), model.expected_tensors(), model.spec.tolerated)
    text = str(error.value)
    assert error.value.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.value.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert "model.layers.0.self_attn.q_proj.weight is [64, 65], expected [64, 64]" in text
    assert "model.layers.0.input_layernorm.weight is torch.int32" in text
    assert "missing tensors (2)" in text and "unexpected tensors (1)" in text


def test_tied_checkpoint_may_still_carry_the_head(tmp_path):
    folder = write_model_folder(tmp_path / "m", "Qwen2ForCausalLM", TINY_A, seed=0)
    tensors = read_all(folder)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    (folder / "model.safetensors").unlink()
    write_file(folder / "model.safetensors", tensors)
    architecture, config = read_model_config(folder)
    model = DecoderModel(architecture.build_spec(config), torch.float32, torch.device("meta"))
    check_tensors(read_model_index(folder), model.expected_tensors(), model.spec.tolerated)


def _raw_file(path, header: dict, payload: bytes):
    text = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(text)) + text + payload)


def test_malformed_safetensors_are_refused(tmp_path):
    path = tmp_path / "x.safetensors"
    path.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError):
        read_header(path)
    path.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError):
        read_header(path)
    _raw_file(path, {"a": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 6]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 8"):
        read_header(path)
    _raw_file(path, {"a": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 8]}}, b"\0" * 4)
    with pytest.raises(SafetensorsError, match="outside the payload"):
        read_header(path)
    _raw_file(path, {"a": {"dtype": "BF16", "shape": [2], "data_offsets": [0, 4]}, "b": {"dtype": "BF16", "shape": [2], "data_offsets": [2, 6]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="overlap"):
        read_header(path)
    _raw_file(path, {"a": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        read_header(path)
    twice = b'{"a":{"dtype":"BF16","shape":[2],"data_offsets":[0,4]},"a":{"dtype":"BF16","shape":[2],"data_offsets":[4,8]}}'
    path.write_bytes(struct.pack("<Q", len(twice)) + twice + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="names 'a' twice"):
        read_header(path)
    _raw_file(path, {"__metadata__": {"format": "pt"}, "a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, struct.pack("<f", 2.5))
    assert read_header(path)["a"].shape == (1,)


def test_sharded_folders_and_their_errors(tmp_path):
    folder = tmp_path / "s"
    folder.mkdir()
    write_file(folder / "p1.safetensors", {"a": torch.ones(3), "b": torch.zeros(2, 2)})
    write_file(folder / "p2.safetensors", {"c": torch.arange(4, dtype=torch.int32)})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "p1.safetensors", "b": "p1.safetensors", "c": "p2.safetensors"}}))
    assert set(read_model_index(folder)) == {"a", "b", "c"}
    assert torch.equal(read_all(folder)["c"], torch.arange(4, dtype=torch.int32))
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "p1.safetensors", "c": "p2.safetensors"}}))
    with pytest.raises(SafetensorsError, match="beyond the index"):
        read_model_index(folder)
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "../p1.safetensors"}}))
    with pytest.raises(SafetensorsError, match="bare file name"):
        read_model_index(folder)
    write_file(folder / "model.safetensors", {"a": torch.ones(1)})
    with pytest.raises(SafetensorsError, match="both"):
        read_model_index(folder)
    with pytest.raises(FileNotFoundError):
        read_model_index(tmp_path / "nothing")


def test_the_config_reader_takes_and_refuses_what_the_reference_reader_does():
    """tests/golden/ignition-config-cases.json holds what the reference's own reader made of 20 documents (made by
    tests/golden/make_config_anchor.py): the same documents are accepted with the same fields, or refused, here."""
    import json
    from pathlib import Path

    from hyperion_b200.config import ConfigError, Qwen2Config

    cases = json.loads((Path(__file__).parent / "golden" / "ignition-config-cases.json").read_text())["cases"]
    assert len(cases) == 20
    for case in cases:
        if "refused" in case:
            with pytest.raises(ConfigError):
                Qwen2Config.from_hf_dict(case["config"])
            continue
        ours, theirs = Qwen2Config.from_hf_dict(case["config"]), case["accepted"]
        assert (ours.num_hidden_layers, ours.hidden_size, ours.intermediate_size, ours.num_attention_heads, ours.num_key_value_heads,
                ours.head_dim, ours.vocab_size, ours.max_position_embeddings, ours.rope_theta, ours.rms_norm_eps, ours.tie_word_embeddings,
                ours.qkv_bias) == (theirs["num_layers"], theirs["hidden_size"], theirs["intermediate_size"], theirs["num_attention_heads"],
                                   theirs["num_kv_heads"], theirs["head_dim"], theirs["vocab_size"], theirs["max_seq_len"], theirs["rope_theta"],
                                   theirs["rms_norm_eps"], theirs["tie_word_embeddings"], theirs["qkv_bias"]), case["name"]


def test_the_reader_returns_the_bytes_the_reference_recorded_for_its_checkpoint():
    """expected.json of the reference's sharded fixture names, for every tensor, its shard, its length in bytes and its
    first and last 16 bytes (the reference checks device bytes against file bytes the same way,
    helios/crates/helios-hal/tests/weights_hw.rs:58): the reader finds every tensor in that shard with those bytes."""
    import json
    from pathlib import Path

    folder = Path(__file__).parent / "golden" / "qwen2-tiny-sharded"
    expected = json.loads((folder / "expected.json").read_text())
    entries = read_model_index(folder)
    tensors = read_all(folder)
    assert set(entries) == set(expected) == set(tensors)
    for name, record in expected.items():
        raw = tensors[name].contiguous().view(torch.uint8).reshape(-1).numpy().tobytes()
        assert entries[name].path.name == record["shard"] and len(raw) == record["length"], name
        assert raw[:16].hex() == record["first16"] and raw[-16:].hex() == record["last16"], name


def test_generation_defaults_follow_the_reference_reader(tmp_path):
    """The same folders give the end-of-sequence ids (config.json first, no repeats) and sampling defaults that the
    reference's ``read_generation`` gave, and what it refused is refused."""
    import json
    from pathlib import Path

    from hyperion_b200.config import ConfigError
    from hyperion_b200.config.generation import GenerationDefaults, read_generation_defaults

    cases = json.loads((Path(__file__).parent / "golden" / "ignition-config-cases.json").read_text())["generation_cases"]
    assert len(cases) == 10
    for index, case in enumerate(cases):
        folder = tmp_path / str(index)
        folder.mkdir()
        (folder / "config.json").write_text(json.dumps(case["config"]))
        if case["generation_config"] is not None:
            (folder / "generation_config.json").write_text(json.dumps(case["generation_config"]))
        if "refused" in case:
            with pytest.raises(ConfigError):
                read_generation_defaults(folder)
            continue
        ours, theirs = read_generation_defaults(folder), case["accepted"]
        assert list(ours.eos_token_ids) == theirs["eos_token_ids"], case["name"]
        defaults = GenerationDefaults()
        for key in ("temperature", "top_p", "top_k", "repetition_penalty"):
            assert getattr(ours, key) == theirs.get("sampling_defaults", {}).get(key, getattr(defaults, key)), (case["name"], key)


def test_expected_tensor_names_and_shapes_are_those_of_the_reference():
    """The reference's table of expected tensors (names by Hugging Face convention, shapes with the hidden size left
    open) for its tiny configuration, tied and untied: the model built from parts expects exactly those."""
    import json
    from pathlib import Path

    cases = json.loads((Path(__file__).parent / "golden" / "ignition-config-cases.json").read_text())["tensor_cases"]
    for case in cases:
        architecture = get_architecture("Qwen2ForCausalLM")
        config = architecture.read_config(case["config"])
        model = DecoderModel(architecture.build_spec(config), torch.float32, torch.device("meta"))
        ours = model.expected_tensors()
        assert set(ours) == set(case["tensors"]), case["name"]
        for name, shape in case["tensors"].items():
            want = tuple(config.hidden_size if extent is None else extent for extent in shape)
            got = tuple(ours[name].shape)
            if name.endswith(("gate_proj.weight", "up_proj.weight")):
                want = (config.intermediate_size, config.hidden_size)  # the reference leaves both extents open
            if name.endswith("down_proj.weight"):
                want = (config.hidden_size, config.intermediate_size)
            assert got == want, (case["name"], name)


def test_the_native_header_reader_on_odd_but_legal_and_on_broken_headers(tmp_path):
    """Names with escapes and non-ASCII letters, metadata of any shape, spaces anywhere, an empty tensor; then headers
    that are not JSON, nest too deeply, or state offsets and extents that are no integers."""
    path = tmp_path / "odd.safetensors"
    header = ('  {"__metadata__": {"note": "a \\"quoted\\" word", "nested": [1, 2.5e3, true, null, {"k": []}]},\n'
              ' "caf\\u00e9/\\ud83d\\ude00": {"dtype": "I32", "shape": [2, 0, 3], "data_offsets": [4, 4]},\t'
              ' "w\u00e4": {"shape": [1], "data_offsets": [0, 4], "dtype": "F32", "extra": "ignored"}}  ').encode("utf-8")
    path.write_bytes(struct.pack("<Q", len(header)) + header + struct.pack("<f", 1.5))
    found = read_header(path)
    assert set(found) == {"caf\u00e9/\U0001f600", "w\u00e4"}
    assert found["caf\u00e9/\U0001f600"].shape == (2, 0, 3) and found["w\u00e4"].dtype == torch.float32
    assert found["w\u00e4"].payload_start == 8 + len(header)

    def refused(text: bytes, payload: bytes = b"\0" * 8) -> str:
        path.write_bytes(struct.pack("<Q", len(text)) + text + payload)
        with pytest.raises(SafetensorsError) as caught:
            read_header(path)
        return str(caught.value)

    assert "not JSON" in refused(b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},}')
    assert "not JSON" in refused(b'{"a": tru}')
    assert "not JSON" in refused(b'{"a": "\x01"}')
    assert "not JSON" in refused(b"[" * 100 + b"]" * 100)
    assert "JSON object" in refused(b'[1, 2]')
    assert "lacks dtype" in refused(b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4.0]}}')
    assert "lacks dtype" in refused(b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [0]}}')
    assert "lacks dtype" in refused(b'{"a": 3}')
    assert "bad shape" in refused(b'{"a": {"dtype": "F32", "shape": [true], "data_offsets": [0, 4]}}')
    assert "bad shape" in refused(b'{"a": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 4]}}')
    assert "needs more than" in refused(b'{"a": {"dtype": "F64", "shape": [4611686018427387904, 4611686018427387904], "data_offsets": [0, 8]}}')
    assert "outside the payload" in refused(b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [-4, 0]}}')
    with pytest.raises(FileNotFoundError):
        read_header(tmp_path / "missing.safetensors")


def test_the_native_header_reader_agrees_with_a_plain_reading_of_written_files(tmp_path):
    import random

    rng = random.Random(5)
    for case in range(20):
        tensors = {}
        for index in range(rng.randrange(1, 12)):
            dtype = rng.choice([torch.bfloat16, torch.float32, torch.int32, torch.uint8, torch.int64])
            shape = [rng.randrange(0, 5) for _ in range(rng.randrange(0, 4))]
            tensors[f"layer.{index}.{'x' * rng.randrange(1, 40)}"] = torch.zeros(shape, dtype=dtype)
        path = tmp_path / f"case{case}.safetensors"
        write_file(path, tensors)
        raw = path.read_bytes()
        (length,) = struct.unpack("<Q", raw[:8])
        plain = json.loads(raw[8 : 8 + length])
        found = read_header(path)
        assert set(found) == set(plain)
        for name, meta in plain.items():
            entry = found[name]
            assert list(entry.shape) == meta["shape"] and [entry.begin, entry.end] == meta["data_offsets"]
            assert entry.payload_start == 8 + length and entry.dtype == tensors[name].dtype


def test_random_weights_are_a_function_of_seed_name_and_index_only(tmp_path):
    """The counter-based generator: Philox4x32-10 as the scalar implementation of the sampler computes it, normal
    deviates of the right moments, a tensor's values independent of which other tensors exist and of how many values are
    asked for, and the same file for the same seed."""
    import numpy as np

    from hyperion_b200.sampling import philox4x32_10 as scalar_philox
    from hyperion_b200.weights import philox_normal
    from hyperion_b200.weights.random_init import random_tensor
    from hyperion_b200.parts.base import WeightSpec

    key = philox_normal.tensor_key(7, "model.layers.0.mlp.up_proj.weight")
    assert key != philox_normal.tensor_key(7, "model.layers.1.mlp.up_proj.weight") != philox_normal.tensor_key(8, "model.layers.1.mlp.up_proj.weight")
    lo = np.array([0, 1, 2 ** 32 - 1, 12345], dtype=np.uint64)
    hi = np.array([0, 0, 3, 2 ** 31], dtype=np.uint64)
    words = philox_normal.philox4x32_10(lo, hi, key)
    for i in range(4):
        assert [int(w[i]) for w in words] == scalar_philox([int(lo[i]), int(hi[i]), 0, 0], list(key))
    values = philox_normal.normal_float32(400_001, key, 1.0)
    assert abs(float(values.mean())) < 0.01 and abs(float(values.std()) - 1.0) < 0.01
    assert abs(float(((values.astype(np.float64)) ** 4).mean()) - 3.0) < 0.1 and 4.0 < float(np.abs(values).max()) < 7.0
    assert 0.67 < float((np.abs(values) < 1.0).mean()) < 0.69
    # a prefix is a prefix (odd and even counts, chunk borders): element i depends on i alone
    assert np.array_equal(philox_normal.normal_float32(33_333, key, 1.0), values[:33_333])
    assert np.array_equal(philox_normal.normal_float32(70_001, key, 1.0, chunk=1000), values[:70_001])
    scaled = philox_normal.normal_float32(1000, key, 0.02, mean=1.0)
    assert abs(float(scaled.mean()) - 1.0) < 0.005 and 0.015 < float(scaled.std()) < 0.025
    tensor = random_tensor("model.layers.0.mlp.up_proj.weight", WeightSpec((10, 40)), 7, 1.0, torch.device("cpu"), torch.bfloat16)
    assert torch.equal(tensor.view(-1), torch.from_numpy(values[:400]).to(torch.bfloat16))
    a = write_model_folder(tmp_path / "a", "Qwen2ForCausalLM", TINY_A, seed=3, device="cpu")
    b = write_model_folder(tmp_path / "b", "Qwen2ForCausalLM", TINY_A, seed=3, device="cpu")
    c = write_model_folder(tmp_path / "c", "Qwen2ForCausalLM", TINY_A, seed=4, device="cpu")
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
