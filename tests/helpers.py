"""Shared pieces of the tests: the two tiny configurations, model folders made in temporary
folders, the plain implementation's logits, and a driver for bin/trace_run."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "tests"))

from plain import qwen2_plain  # noqa: E402

from hyperion_b200.config import Qwen2Config  # noqa: E402
from hyperion_b200.weights import write_model_folder  # noqa: E402

# Two tiny configurations that differ in every size and option: heads and groups, head size, widths
# that are no power of two, layers, vocabulary, eps, RoPE base, tied or untied head.
TINY_A = Qwen2Config(num_hidden_layers=2, hidden_size=64, intermediate_size=176, num_attention_heads=4, num_key_value_heads=2,
                     head_dim=16, vocab_size=256, max_position_embeddings=512, rope_theta=10000.0, rms_norm_eps=1e-6,
                     tie_word_embeddings=True)
TINY_B = Qwen2Config(num_hidden_layers=3, hidden_size=192, intermediate_size=400, num_attention_heads=6, num_key_value_heads=1,
                     head_dim=32, vocab_size=523, max_position_embeddings=1024, rope_theta=1e6, rms_norm_eps=1e-5,
                     tie_word_embeddings=False)
# A third one whose head size (64) and page size take the TMA-fed attention kernels; A and B (16, 32) take the cp.async ones.
TINY_C = Qwen2Config(num_hidden_layers=2, hidden_size=256, intermediate_size=264, num_attention_heads=4, num_key_value_heads=2,
                     head_dim=64, vocab_size=300, max_position_embeddings=512, rope_theta=50000.0, rms_norm_eps=1e-6,
                     tie_word_embeddings=False)
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2)}
WEIGHT_STD = 0.06  # larger than an initialiser's 0.02 so that attention is peaked and logits are O(1)
# The two tiny configurations as the benchmark file states them, sizes and N(0, 0.02) weights and all.  A and B above are
# harder versions of them (a vocabulary and an intermediate size that are no power of two, longer positions, weights
# three times as large so that logits are O(1) and attention is peaked); these run their stated workloads once.
STATED_A = Qwen2Config(num_hidden_layers=2, hidden_size=64, intermediate_size=176, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=16, vocab_size=256, max_position_embeddings=128, rope_theta=10000.0, rms_norm_eps=1e-6,
                       tie_word_embeddings=True)
STATED_B = Qwen2Config(num_hidden_layers=3, hidden_size=192, intermediate_size=384, num_attention_heads=6, num_key_value_heads=1,
                       head_dim=32, vocab_size=512, max_position_embeddings=256, rope_theta=1e6, rms_norm_eps=1e-5,
                       tie_word_embeddings=False)
STATED = {"A": (STATED_A, 0), "B": (STATED_B, 1)}
STATED_STD = 0.02

# Declared before the first run. float32: the engine's fixed-order float arithmetic against the
# plain float64 implementation. bfloat16: a few roundings to 8 bits of mantissa (2^-9 relative
# each) through the layers, against the same float64 reference on the same bfloat16 weights.
TOLERANCE = {"float32": 2e-5, "bfloat16": 2.5e-2}


def make_folder(tmp: Path, name: str, std: float = WEIGHT_STD) -> Path:
    config, seed = TINY[name]
    return write_model_folder(Path(tmp) / f"tiny_{name}", "Qwen2ForCausalLM", config, seed, std)


def make_stated_folder(tmp: Path, name: str) -> Path:
    config, seed = STATED[name]
    return write_model_folder(Path(tmp) / f"stated_{name}", "Qwen2ForCausalLM", config, seed, STATED_STD)


def plain_logits(folder: Path, ids, device: str = "cpu") -> np.ndarray:
    """The plain implementation's float64 logits of one whole sequence; ``device`` is where torch does that arithmetic."""
    config, weights = qwen2_plain.read_model_folder(folder)
    return qwen2_plain.forward(config, weights, list(ids), device=device).cpu().numpy()


def random_ids(seed: int, count: int, vocab: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=generator).tolist()


def run_trace(folder: Path, dtype: str, steps: list[dict], out: Path, max_tokens: int, page_size: int = 16, env: dict | None = None,
              pages_log: Path | None = None) -> dict[int, np.ndarray]:
    """Feed ``steps`` to bin/trace_run and read back the logits of every step that wanted some."""
    out = Path(out)
    out.mkdir(parents=True, exist_ok=True)
    text = "".join(json.dumps(step) + "\n" for step in steps)
    command = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
               "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
    if pages_log is not None:
        command += ["--pages-log", str(pages_log)]
    done = subprocess.run(command, input=text, capture_output=True, text=True, timeout=900, env={**os.environ, **(env or {})})
    assert done.returncode == 0, f"trace_run failed:\n{done.stdout[-2000:]}\n{done.stderr[-4000:]}"
    finished = [line for line in done.stdout.splitlines() if line.startswith("done ")]
    assert [int(line.split()[1]) for line in finished] == [s["step"] for s in steps]
    config = json.loads((Path(folder) / "config.json").read_text())
    results = {}
    for step in steps:
        wanted = sum(len(e.get("want", ())) for e in step["entries"])
        if wanted:
            data = np.fromfile(out / f"{step['step']}.f32", dtype="<f4")
            results[step["step"]] = data.reshape(wanted, config["vocab_size"])
    return results


def compare_steps(steps: list[dict], results: dict[int, np.ndarray], reference: dict[str, np.ndarray], tolerance: float) -> float:
    """Every wanted position of every step against the plain logits of its request; returns the
    worst error relative to the largest reference logit of its row."""
    fed: dict[str, int] = {}
    worst = 0.0
    for step in steps:
        row = 0
        for entry in step["entries"]:
            start = fed.get(entry["id"], 0)
            for index in entry.get("want", ()):
                got = results[step["step"]][row]
                want = reference[entry["id"]][start + index]
                scale = max(1e-6, float(np.abs(want).max()))
                error = float(np.abs(got - want).max()) / scale
                assert np.isfinite(got).all(), f"step {step['step']} request {entry['id']} position {start + index}: not finite"
                assert error <= tolerance, (f"step {step['step']} request {entry['id']} position {start + index}: "
                                            f"relative error {error:.3e} above {tolerance:.1e}")
                worst = max(worst, error)
                row += 1
            fed[entry["id"]] = start + len(entry["tokens"])
        for request in step.get("end", ()):
            fed.pop(request, None)
    return worst


def logits_by_position(steps: list[dict], results: dict[int, np.ndarray]) -> dict[tuple[str, int], np.ndarray]:
    """{(request, position): its logits row} of a replayed trace."""
    fed: dict[str, int] = {}
    rows = {}
    for step in steps:
        row = 0
        for entry in step["entries"]:
            start = fed.get(entry["id"], 0)
            for index in entry.get("want", ()):
                rows[(entry["id"], start + index)] = results[step["step"]][row]
                row += 1
            fed[entry["id"]] = start + len(entry["tokens"])
        for request in step.get("end", ()):
            fed.pop(request, None)
    return rows


def check_pages_log(path: Path, steps: list[dict], pool_pages: int) -> dict:
    """Replays a page log: no page is ever in two tables, a page given back was held by the request that gives it,
    nothing is held at the end.  Returns how many pages changed owner."""
    held: dict[tuple[int, int], str] = {}  # (group, page) -> request
    last_owner: dict[tuple[int, int], str] = {}
    handed_on = 0
    records = [json.loads(line) for line in Path(path).read_text().splitlines()]
    assert [r["step"] for r in records] == [s["step"] for s in steps]
    for record in records:
        for request, group, block, page in record["taken"]:
            assert 0 <= page < pool_pages and (group, page) not in held, f"step {record['step']}: page {page} of group {group} is held twice"
            held[(group, page)] = request
            if last_owner.get((group, page), request) != request:
                handed_on += 1
        for request, group, block, page in record["returned"]:
            assert held.get((group, page)) == request, f"step {record['step']}: {request} gives back page {page} it does not hold"
            del held[(group, page)]
            last_owner[(group, page)] = request
    assert not held, f"pages still held at the end: {held}"
    return {"handed_on": handed_on, "pages_used": len(last_owner)}
