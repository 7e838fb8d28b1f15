"""Makes the anchor of the plain implementation: the reference's committed tiny checkpoint and the
float32 oracle that was computed for it.

The reference's model code is Rust and CUDA and cannot be compiled or run on a machine without its
toolchain, but the repository commits a tiny random Qwen2 checkpoint
(testdata/synthetic/qwen2-tiny-sharded, made by scripts/gen-sharded-fixture.py:32-50) and, for it,
float32 top-20 logits and logsumexp at 16 teacher-forced positions of four prompts
(testdata/oracle/qwen2-tiny-sharded.compact.json, compared by the rule of
helios/crates/helios-hal/src/oracle.rs:197-217).  This script copies the checkpoint's files and
cuts the oracle down to what the tests read: per position the float32 record and how far the
reference's own bfloat16 run was from it there (``bf16_deviation``, the width of the tie group in
oracle.rs:197-217), and the largest such distance over all positions (``bf16_vs_fp32``).

    python tests/golden/make_anchor.py /path/to/reference

Outputs (committed): tests/golden/qwen2-tiny-sharded/ (with the reference's expected.json: shard, length and first
and last 16 bytes of every tensor, written by scripts/gen-sharded-fixture.py:59-66) and tests/golden/qwen2-tiny-oracle.json.
"""
import json
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def main(reference: Path) -> None:
    source = reference / "testdata" / "synthetic" / "qwen2-tiny-sharded"
    target = HERE / "qwen2-tiny-sharded"
    target.mkdir(exist_ok=True)
    for path in sorted(source.iterdir()):
        if path.suffix == ".safetensors" or path.name in ("config.json", "model.safetensors.index.json", "expected.json"):
            shutil.copyfile(path, target / path.name)
    oracle = json.loads((reference / "testdata" / "oracle" / "qwen2-tiny-sharded.compact.json").read_text())
    prompts = []
    for prompt in oracle["prompts"]:
        prompts.append({"ids": prompt["ids"], "generated_ids": prompt["generated_ids"],
                        "positions": [{k: row[k] for k in ("position", "argmax", "top_ids", "top_logits", "logsumexp")}
                                      for row in prompt["reference_fp32"]],
                        "bf16_deviation": [row["top_logits"] for row in prompt["bf16_deviation"]]})
    document = {"source": "testdata/oracle/qwen2-tiny-sharded.compact.json of the reference", "format": oracle["format"],
                "tolerance": {k: oracle["tolerance"][k] for k in ("max_abs_top_logits", "max_abs_logsumexp")},
                "bf16_vs_fp32": {k: oracle["bf16_vs_fp32"][k] for k in ("top_logits", "logsumexp")}, "prompts": prompts}
    (HERE / "qwen2-tiny-oracle.json").write_text(json.dumps(document))


if __name__ == "__main__":
    main(Path(sys.argv[1]))
