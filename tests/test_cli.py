"""The command line: the ``random`` command without a GPU, ``generate`` on one."""
from __future__ import annotations

import json
import subprocess
import sys

import pytest

from helpers import ROOT, TINY_A


def run_cli(*args, **kw):
    return subprocess.run([sys.executable, "-m", "hyperion_b200", *args], cwd=ROOT, capture_output=True, text=True, timeout=600, **kw)


def test_random_command_writes_a_loadable_folder(tmp_path):
    from hyperion_b200.models import read_model_config
    from hyperion_b200.weights import read_model_index

    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(TINY_A.to_hf_dict()))
    done = run_cli("random", "--config", str(config_path), "--out", str(tmp_path / "model"), "--seed", "4")
    assert done.returncode == 0, done.stderr
    assert json.loads(done.stdout)["written"].endswith("model")
    _, config = read_model_config(tmp_path / "model")
    assert config == TINY_A and len(read_model_index(tmp_path / "model")) == 26


def test_option_names_follow_the_reference():
    from hyperion_b200.cli import build_parser

    args = build_parser().parse_args(["generate", "-m", "x", "--prompt-ids", "1,2 3", "--max-seq-len", "64", "--max-batch", "4",
                                      "--default-max-tokens", "9", "--prefill-chunk-busy", "128", "--temperature", "0", "--top-p", "0.9",
                                      "--top-k", "5", "--repetition-penalty", "1.1", "--seed", "3", "--max-tokens", "7"])
    assert (args.model, args.max_seq_len, args.max_batch, args.default_max_tokens, args.prefill_chunk_busy) == ("x", 64, 4, 9, 128)
    assert (args.temperature, args.top_p, args.top_k, args.repetition_penalty, args.seed, args.max_tokens) == (0.0, 0.9, 5, 1.1, 3, 7)


@pytest.mark.gpu
def test_generate_command_matches_the_plain_greedy_continuation(tmp_path):
    from plain import qwen2_plain

    from hyperion_b200.weights import write_model_folder

    folder = write_model_folder(tmp_path / "m", "Qwen2ForCausalLM", TINY_A, seed=0, std=0.06)
    done = run_cli("generate", "-m", str(folder), "--dtype", "float32", "--prompt-ids", "5,17,3,9", "--prompt-ids", "200 1", "--temperature", "0",
                   "--max-tokens", "5", "--max-seq-len", "64", "--ignore-eos")
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    config, weights = qwen2_plain.read_model_folder(folder)
    assert [line["tokens"] for line in lines] == [qwen2_plain.greedy(config, weights, p, 5) for p in ([5, 17, 3, 9], [200, 1])]
    assert all(line["finish_reason"] == "length" for line in lines)
    bad = run_cli("generate", "-m", str(folder), "--prompt-ids", "1", "--max-seq-len", "100000")
    assert bad.returncode == 2 and "--max-seq-len" in bad.stderr
