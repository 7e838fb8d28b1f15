"""Command line: ``python -m hyperion_b200 <command>``.

``generate`` loads a model folder and continues prompts given as token ids; ``random`` writes a
model folder with seeded random weights from a config.json.  Option names and meanings follow the
reference's launcher where it has them (helios/crates/helios-cli/src/main.rs:44-87): ``-m/--model``,
``--max-seq-len`` (longest prompt + generation, at most the model's), ``--max-batch`` (most
sequences decoded together), ``--default-max-tokens`` (for a request without ``--max-tokens``),
``--prefill-chunk-busy`` (largest prompt portion while sequences are decoding); and its request
fields ``temperature``, ``top_p``, ``top_k``, ``repetition_penalty``, ``seed``, ``max_tokens``
(helios/crates/helios-core/src/api.rs:111-124).  The reference serves HTTP and has no tokenizer-free
entry; this engine starts at token ids, so prompts are lists of ids.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def _ids(text: str) -> list[int]:
    return [int(piece) for piece in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="hyperion_b200", description="Single-GPU inference engine for sm_100a")
    commands = parser.add_subparsers(dest="command", required=True)

    g = commands.add_parser("generate", help="continue prompts given as token ids")
    g.add_argument("-m", "--model", required=True, help="folder with config.json and safetensors")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--prompt-ids", action="append", default=[], help="token ids separated by commas or spaces; repeatable")
    g.add_argument("--prompts-file", help="file with one JSON list of token ids per line")
    g.add_argument("--max-seq-len", type=int, default=None, help="longest sequence (prompt + generation); defaults to the model's")
    g.add_argument("--max-batch", type=int, default=32, help="most sequences decoded together in one step")
    g.add_argument("--default-max-tokens", type=int, default=1024, help="max_tokens of a request that states none")
    g.add_argument("--prefill-chunk-busy", type=int, default=512, help="largest prompt portion, in tokens, while sequences are decoding")
    g.add_argument("--max-batch-tokens", type=int, default=2048, help="token budget of one step")
    g.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    g.add_argument("--cache-tokens", type=int, default=None, help="tokens the cache holds; default max-batch * max-seq-len")
    g.add_argument("--max-tokens", type=int, default=None)
    g.add_argument("--temperature", type=float, default=None, help="0 is greedy")
    g.add_argument("--top-p", type=float, default=None)
    g.add_argument("--top-k", type=int, default=None, help="0 keeps the whole vocabulary")
    g.add_argument("--repetition-penalty", type=float, default=None)
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--ignore-eos", action="store_true")

    r = commands.add_parser("random", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="a config.json naming the architecture and its sizes")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=0.02)
    return parser


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.command == "random":
        from .config.base import read_json
        from .models import architecture_of
        from .weights import write_model_folder

        document = read_json(Path(args.config))
        architecture = architecture_of(document)
        folder = write_model_folder(Path(args.out), architecture.name, architecture.read_config(document), args.seed, args.std)
        print(json.dumps({"written": str(folder)}))
        return 0

    from .api import Engine
    from .models import read_model_config
    from .sampling import SamplingParams

    prompts = [_ids(text) for text in args.prompt_ids]
    if args.prompts_file:
        with open(args.prompts_file, "r", encoding="utf-8") as handle:
            prompts += [json.loads(line) for line in handle if line.strip()]
    if not prompts:
        print("no prompts: give --prompt-ids or --prompts-file", file=sys.stderr)
        return 2
    _, config = read_model_config(Path(args.model))
    limit = getattr(config, "max_position_embeddings", None)
    max_seq_len = args.max_seq_len or limit
    if limit is not None and not 0 < max_seq_len <= limit:
        print(f"--max-seq-len {max_seq_len} is outside 1..={limit} (the model's max_seq_len): choose a value in that range", file=sys.stderr)
        return 2
    cache_tokens = args.cache_tokens or min(args.max_batch, len(prompts)) * max_seq_len
    engine = Engine.from_folder(args.model, dtype=args.dtype, page_size=args.page_size, max_tokens=cache_tokens, max_requests=args.max_batch)
    d = engine.defaults
    temperature = d.temperature if args.temperature is None else args.temperature
    params = SamplingParams(
        temperature=temperature, top_p=d.top_p if args.top_p is None else args.top_p, top_k=d.top_k if args.top_k is None else args.top_k,
        # greedy decoding cannot apply a penalty: one that only comes from the defaults is dropped
        repetition_penalty=(1.0 if temperature == 0 else d.repetition_penalty) if args.repetition_penalty is None else args.repetition_penalty,
        seed=args.seed, max_tokens=args.max_tokens or args.default_max_tokens, ignore_eos=args.ignore_eos)
    outputs, reasons = engine.generate(prompts, params, max_batch=args.max_batch, max_batch_tokens=args.max_batch_tokens,
                                       prefill_chunk_busy=args.prefill_chunk_busy, max_seq_len=max_seq_len, return_reasons=True)
    for index, (tokens, reason) in enumerate(zip(outputs, reasons)):
        print(json.dumps({"index": index, "tokens": tokens, "finish_reason": reason}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
