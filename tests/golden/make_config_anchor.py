"""Runs the reference's own config reader on a set of config.json documents and records what it makes of each.

The reference's build-time package is plain Python (ignition/src/hyperion_ignition); its
``model_config_from_hf`` (compiler/model_config.py:95-169) is what decides which Qwen2 configurations it takes and
what the fields mean.  This script imports it from a checkout of the reference, feeds it the reference's own two
configurations (testdata/synthetic/qwen2-tiny-sharded/config.json, ignition/tests/fixtures/qwen2-hf/config.json) and
variants of them (defaults left out, the nested rope form, every refusal), and writes the documents with the outcomes:

    python tests/golden/make_config_anchor.py /path/to/reference

Output (committed): tests/golden/ignition-config-cases.json.  ``tests/test_config_weights.py`` holds this
package's reader to the same outcomes.
"""
import dataclasses
import json
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent


def variants(tiny: dict, large: dict) -> list[tuple[str, dict]]:
    def changed(base, **changes):
        document = dict(base)
        for key, value in changes.items():
            if value is None:
                document.pop(key, None)
            else:
                document[key] = value
        return document

    nested = changed(large, rope_theta=None, rope_parameters={"rope_theta": 500000.0, "rope_type": "default"})
    return [
        ("the reference's tiny checkpoint", tiny),
        ("the reference's 7B fixture", large),
        ("head_dim stated", changed(large, head_dim=128)),
        ("head_dim unlike hidden / heads", changed(tiny, head_dim=32)),
        ("no num_key_value_heads", changed(tiny, num_key_value_heads=None)),
        ("rope_theta nested in rope_parameters", nested),
        ("tied embeddings", changed(tiny, tie_word_embeddings=True)),
        ("rope_scaling set", changed(large, rope_scaling={"type": "yarn", "factor": 4.0})),
        ("rope_scaling null", changed(large, rope_scaling=None) | {"rope_scaling": None}),
        ("use_sliding_window true", changed(large, use_sliding_window=True)),
        ("hidden_act gelu", changed(large, hidden_act="gelu")),
        ("partial rotary", changed(large, partial_rotary_factor=0.5)),
        ("tie_word_embeddings missing", changed(large, tie_word_embeddings=None)),
        ("rms_norm_eps missing", changed(large, rms_norm_eps=None)),
        ("rope_theta missing", changed(large, rope_theta=None)),
        ("kv heads do not divide heads", changed(large, num_key_value_heads=5)),
        ("hidden not divisible by heads", changed(tiny, hidden_size=66)),
        ("another architecture", changed(large, architectures=["LlamaForCausalLM"])),
        ("vocab_size zero", changed(large, vocab_size=0)),
        ("num_hidden_layers a string", changed(large, num_hidden_layers="28")),
    ]


def main(reference: Path) -> None:
    sys.path.insert(0, str(reference / "ignition" / "src"))
    from hyperion_ignition.compiler.model_config import model_config_from_hf

    tiny = json.loads((reference / "testdata" / "synthetic" / "qwen2-tiny-sharded" / "config.json").read_text())
    large = json.loads((reference / "ignition" / "tests" / "fixtures" / "qwen2-hf" / "config.json").read_text())
    cases = []
    for name, document in variants(tiny, large):
        with tempfile.TemporaryDirectory() as folder:
            (Path(folder) / "config.json").write_text(json.dumps(document))
            try:
                config = model_config_from_hf(Path(folder), ("Qwen2ForCausalLM",), qkv_bias=True)
                outcome = {"accepted": dataclasses.asdict(config)}
            except (ValueError, KeyError, TypeError, FileNotFoundError) as error:
                outcome = {"refused": f"{type(error).__name__}: {error}"}
        cases.append({"name": name, "config": document, **outcome})
    from hyperion_ignition.compiler.generation import read_generation

    generation_cases = []
    for name, config_eos, generation in [
        ("one id in config.json", 7, None),
        ("a list in generation_config.json", None, {"eos_token_id": [3, 9]}),
        ("both, overlapping: config first, no repeats", [9, 4], {"eos_token_id": [3, 9, 4, 11]}),
        ("sampling defaults", 7, {"temperature": 0.7, "top_p": 0.8, "top_k": 20, "repetition_penalty": 1.05}),
        ("some sampling defaults, top_k as a float", 7, {"temperature": 0.6, "top_k": 20.0}),
        ("null values are left out", 7, {"temperature": None, "top_p": 0.9}),
        ("a negative value", 7, {"temperature": -1.0}),
        ("a boolean value", 7, {"top_p": True}),
        ("a negative id", -2, None),
        ("a boolean id", None, {"eos_token_id": [True]}),
    ]:
        document = dict(large)
        document.pop("eos_token_id", None)
        if config_eos is not None:
            document["eos_token_id"] = config_eos
        with tempfile.TemporaryDirectory() as folder:
            (Path(folder) / "config.json").write_text(json.dumps(document))
            if generation is not None:
                (Path(folder) / "generation_config.json").write_text(json.dumps(generation))
            try:
                outcome = {"accepted": read_generation(Path(folder))}
            except (ValueError, KeyError, TypeError) as error:
                outcome = {"refused": f"{type(error).__name__}: {error}"}
        generation_cases.append({"name": name, "config": document, "generation_config": generation, **outcome})
    from hyperion_ignition.compiler.weights import _qwen2_expected

    tensor_cases = []
    for name, document in (("the reference's tiny checkpoint (untied)", tiny), ("tied", dict(tiny, tie_word_embeddings=True))):
        with tempfile.TemporaryDirectory() as folder:
            (Path(folder) / "config.json").write_text(json.dumps(document))
            config = model_config_from_hf(Path(folder), ("Qwen2ForCausalLM",), qkv_bias=True)
        expected = _qwen2_expected(config, document["tie_word_embeddings"])
        tensor_cases.append({"name": name, "config": document, "tensors": {k: list(v) for k, v in expected.items()}})
    (HERE / "ignition-config-cases.json").write_text(json.dumps({
        "source": "model_config_from_hf and read_generation of the reference (ignition/src/hyperion_ignition/compiler/model_config.py:95-169, "
                  "generation.py:51-71)", "cases": cases, "generation_cases": generation_cases,
        "tensor_cases": tensor_cases, "tensor_source": "_qwen2_expected (compiler/weights.py:175-207): names and shapes, null = the hidden size"}, indent=1))
    print(f"{sum('accepted' in c for c in cases)} accepted, {sum('refused' in c for c in cases)} refused; generation: "
          f"{sum('accepted' in c for c in generation_cases)} accepted, {sum('refused' in c for c in generation_cases)} refused")


if __name__ == "__main__":
    main(Path(sys.argv[1]))
