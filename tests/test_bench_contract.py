"""What ``bench.py`` promises without a GPU: its refusal of more than one GPU, the reference arm's line, and the
arithmetic behind the figures it prints (bytes a decode step has to read, operations of a prompt step, percentiles)."""
from __future__ import annotations

import importlib.util
import json
import subprocess
import sys

from helpers import ROOT


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def run_bench(*args, env=None):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], cwd=ROOT, capture_output=True, text=True, timeout=300, env=env)


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    done = run_bench("--gpus", "2", "--steps", "3", "--warmup", "1")
    assert done.returncode == 2
    assert len(done.stdout.strip().splitlines()) == 1 and "one GPU" in done.stdout


def test_the_reference_arm_says_why_it_is_unavailable():
    done = run_bench("--impl", "reference", "--gpus", "1", "--steps", "3", "--warmup", "1")
    assert done.returncode == 0
    lines = done.stdout.strip().splitlines()
    assert len(lines) == 1
    record = json.loads(lines[0])
    assert record["impl"] == "reference" and isinstance(record["unavailable"], str) and record["unavailable"]


def test_weight_bytes_and_prompt_operations_follow_the_configuration():
    bench = load_bench()
    config = bench.model_config(28)
    hidden, inter, vocab = config.hidden_size, config.intermediate_size, config.vocab_size
    q, kv = config.num_attention_heads * config.head_dim, config.num_key_value_heads * config.head_dim
    # every matrix a decode step multiplies by, once, in bfloat16 (biases too), and the norms' float weights; the embedding
    # table is only looked up in
    matrices = 28 * ((q + 2 * kv) * hidden + (q + 2 * kv) + q * hidden + 3 * hidden * inter) + vocab * hidden
    assert bench.weight_bytes(config) == 2 * matrices + 4 * (2 * 28 + 1) * hidden
    assert 14.1e9 < bench.weight_bytes(config) < 14.2e9
    # a prompt of T tokens: two operations per weight and token, causal attention over T (T + 1) / 2 pairs, the head once
    tokens = 2048
    linear = 2.0 * tokens * ((q + 2 * kv) * hidden + q * hidden + 3 * hidden * inter)
    attention = 4.0 * q * tokens * (tokens + 1) / 2
    assert bench.prefill_flops(config, tokens) == 28 * (linear + attention) + 2.0 * hidden * vocab
    fewer = bench.model_config(2)
    assert bench.weight_bytes(fewer) < bench.weight_bytes(config) / 5


def test_percentiles_interpolate_between_neighbours():
    bench = load_bench()
    values = [5.0, 1.0, 3.0, 2.0, 4.0]
    assert bench.percentile(values, 0.0) == 1.0 and bench.percentile(values, 1.0) == 5.0
    assert bench.percentile(values, 0.5) == 3.0
    assert abs(bench.percentile(values, 0.1) - 1.4) < 1e-12 and abs(bench.percentile(values, 0.9) - 4.6) < 1e-12
    assert bench.percentile([7.0], 0.9) == 7.0


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    bench = load_bench()
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    peaks, source = bench.peaks()
    assert source == "fallback" and peaks == bench.FALLBACK_PEAKS
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6000.0, "bf16_tflops": 1500.0, "bf16_tflops_sustained": 1300.0}))
    peaks, source = bench.peaks()
    assert source == "measured" and peaks["hbm_gbs"] == 6000.0
