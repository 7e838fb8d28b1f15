"""Decode and prefill throughput of the engine on one B200, Qwen2.5-7B shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

Prints ONE JSON line.  Every decode figure is taken over the whole range the configuration names: ``batch``
requests are each prefilled with 2,048 random token ids and then decoded to a context of 4,096 (one new token per
request per step, output head and token choice included).  After W untimed steps the rest of the range is timed in
windows of exactly K steps, a CUDA event between every two windows (at least ten windows: K is capped at a tenth of
the range).  ``value`` is decoded tokens per second over all windows at the given batch (default 8), ``ms_per_step``
the same as time per step; ``windows`` gives the median, the 10th and the 90th percentile of the windows' time per
step and the rate of the windows at contexts of about 2,048, 3,072 and 4,096 (the reference's protocol: at least ten
windows, median [p10, p90], docs/performance-log.md:5).  ``points`` holds the same whole-range figure at batch 1 and
64.  ``e2e`` is the same range through ``Engine.generate`` (token ids in from the host, sampled ids back to the host
every step), timed on the host.  ``prefill`` is one whole 2,048-token prompt in one step (from its third occurrence on
the engine replays a step shape from a captured graph, as it does for decode steps; the timed repetitions are such
replays): timed first, on an idle GPU, as a burst against the burst peak, and once more at the end as the median of
20 repetitions under sustained load (``sustained_*``, against the sustained peak: the board's power cap lowers the
clocks within a few hundred milliseconds of such steps).  ``roofline`` relates the decode step to the bytes it has to read (every weight it uses once, plus the
cache of the live requests at the mean context of the timed steps).  Weights (15 GB) are larger than L2, so every
step streams them from HBM.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT = 2048
CONTEXT = 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# What the reference publishes for this model: decode by batch on one H100 at context 512 (docs/performance-log.md:239-242).
# It has no number on a B200, none at contexts of 2,048 to 4,096 by batch, and none at batch 64.
BASELINE_TOK_S = {1: 146.0, 8: 1087.0}
BASELINE_LABEL = {"gpu": "H100 80GB", "context": 512, "unit": "tokens/s", "source": "docs/performance-log.md:239-242 of the reference"}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.path = Path(tempfile.mkstemp(suffix=".csv")[1])
        self.process = None

    def start(self):
        try:
            self.process = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                                            stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.path.read_text().splitlines():
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 6:
                continue
            try:
                clocks.append(float(fields[0]))
                maxima.append(float(fields[1]))
            except ValueError:
                continue
            for name, value in zip(names, fields[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        self.path.unlink(missing_ok=True)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(maxima) if maxima else None,
                "reasons": sorted(reasons)}


def reference_arm() -> int:
    # The reference's runtime is Rust (helios) with CUDA kernels built for sm_80/sm_90; this image has
    # no cargo or rustc, and pip finds no Python project at the root of the reference's tree.
    print(json.dumps({"impl": "reference", "unavailable": "the reference runtime is Rust + sm_90 CUDA; no Rust toolchain in this image and pip finds no installable project at its root"}))
    return 0


def model_config(layers: int):
    from hyperion_b200.config import Qwen2Config

    return Qwen2Config(num_hidden_layers=layers, hidden_size=3584, intermediate_size=18944, num_attention_heads=28,
                       num_key_value_heads=4, head_dim=128, vocab_size=152064, max_position_embeddings=32768, rope_theta=1e6,
                       rms_norm_eps=1e-6, tie_word_embeddings=False)


def weight_bytes(c) -> int:
    q, kv = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
    per_layer = (q + 2 * kv) * c.hidden_size + (q + 2 * kv) + q * c.hidden_size + 3 * c.hidden_size * c.intermediate_size
    return 2 * (c.num_hidden_layers * per_layer + c.vocab_size * c.hidden_size) + 4 * (2 * c.num_hidden_layers + 1) * c.hidden_size


def prefill_flops(c, tokens: int) -> float:
    q, kv = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
    linear = 2.0 * tokens * ((q + 2 * kv) * c.hidden_size + q * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
    attention = 4.0 * c.num_attention_heads * c.head_dim * tokens * (tokens + 1) / 2
    return c.num_hidden_layers * (linear + attention) + 2.0 * c.hidden_size * c.vocab_size


def random_prompt(seed: int, count: int, vocab: int) -> list[int]:
    import torch

    return torch.randint(0, vocab, (count,), generator=torch.Generator().manual_seed(seed)).tolist()


def percentile(values: list[float], fraction: float) -> float:
    ordered = sorted(values)
    at = fraction * (len(ordered) - 1)
    low = int(at)
    high = min(low + 1, len(ordered) - 1)
    return ordered[low] + (ordered[high] - ordered[low]) * (at - low)


def time_decode(engine, batch: int, window: int, warmup: int, decode_tokens: int = CONTEXT - PROMPT) -> dict:
    """``batch`` requests prefilled to 2,048 tokens and decoded by ``decode_tokens`` more: W untimed steps, then windows
    of exactly ``window`` steps with a CUDA event between every two, to the end of the range."""
    import torch

    from hyperion_b200.engine.batch import StepEntry
    from hyperion_b200.ops import native
    from hyperion_b200.sampling import GREEDY, pack_options

    vocab = engine.model.spec.vocab_size
    names = [f"bench{batch}_{i}" for i in range(batch)]
    for i, name in enumerate(names):
        engine.step([StepEntry(name, random_prompt(i, PROMPT, vocab), [])])
    window = max(1, min(window, (decode_tokens - warmup) // 10))
    n_windows = (decode_tokens - warmup) // window
    steps = n_windows * window
    feed = torch.randint(0, vocab, (warmup + steps, batch), generator=torch.Generator().manual_seed(1000 + batch)).tolist()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(n_windows + 1)]
    options = {"sampling_options": ([w for name in names for w in pack_options(GREEDY, 0, engine.cache.slot(name))], (batch, 8))}

    def one(s):
        logits = engine.runner.step([StepEntry(name, [feed[s][i]], [0]) for i, name in enumerate(names)], options)
        engine.sampler.sample(logits, engine.runner.last_context.extra["sampling_options"], all_greedy=True)

    for s in range(warmup):
        one(s)
    torch.cuda.synchronize()
    launches_before = native.LAUNCHES[0] + getattr(engine.runner, "graph_launches", 0)
    host_start = time.perf_counter()
    events[0].record()
    for w in range(n_windows):
        for s in range(warmup + w * window, warmup + (w + 1) * window):
            one(s)
        events[w + 1].record()
    torch.cuda.synchronize()
    host_ms = (time.perf_counter() - host_start) * 1e3
    per_window = [events[w].elapsed_time(events[w + 1]) / window for w in range(n_windows)]  # ms per step
    ms = events[0].elapsed_time(events[-1])
    launches = native.LAUNCHES[0] + getattr(engine.runner, "graph_launches", 0) - launches_before
    mean_context = PROMPT + warmup + (steps + 1) / 2
    h2d = engine.runner.packer._cursor * 4
    for name in names:
        engine.finish(name)
    engine.check()

    def rate_at(context: int) -> float:
        index = min(n_windows - 1, max(0, (context - PROMPT - warmup) // window))
        return round(batch / (per_window[index] / 1e3), 1)

    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "host_ms_per_step": host_ms / steps,
            "launches": launches, "mean_context": mean_context, "h2d_bytes": h2d, "steps": steps, "window": window,
            "windows": {"count": n_windows, "steps_each": window, "ms_per_step_median": round(statistics.median(per_window), 4),
                        "ms_per_step_p10": round(percentile(per_window, 0.1), 4), "ms_per_step_p90": round(percentile(per_window, 0.9), 4),
                        "tokens_per_s_at_context": {str(c): rate_at(c) for c in (PROMPT, (PROMPT + PROMPT + decode_tokens) // 2, PROMPT + decode_tokens)}}}


def time_prefill(engine, reps: int = 5, warmup: int = 3) -> dict:
    import torch

    from hyperion_b200.engine.batch import StepEntry

    vocab = engine.model.spec.vocab_size
    times = []
    for r in range(warmup + reps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        prompt = random_prompt(50 + r, PROMPT, vocab)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry("prefill", prompt, [PROMPT - 1])])
        stop.record()
        torch.cuda.synchronize()
        engine.finish("prefill")
        if r >= warmup:
            times.append(start.elapsed_time(stop))
    engine.check()
    return {"ms": statistics.median(times)}


def time_e2e(engine, batch: int, window: int, warmup: int, decode_tokens: int = CONTEXT - PROMPT) -> dict:
    """The same range through ``Engine.generate``: prompts go in from the host; every step copies its metadata from
    pinned memory and its sampled ids back to pinned memory, where the callback reads them (one step behind the device,
    which takes each token from the step before on the device).  Timed on the host, from the W-th token of the last
    request to its last token."""
    from hyperion_b200.sampling import SamplingParams

    vocab = engine.model.spec.vocab_size
    prompts = [random_prompt(i, PROMPT, vocab) for i in range(batch)]
    stamps: list[float] = []

    def on_token(index, token):
        if index == batch - 1:
            stamps.append(time.perf_counter())

    engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=decode_tokens, ignore_eos=True), max_batch=batch,
                    max_batch_tokens=batch * PROMPT, prefill_chunk_busy=PROMPT, on_token=on_token)
    steps = len(stamps) - 1 - warmup
    seconds = stamps[-1] - stamps[warmup]
    window = max(1, min(window, steps // 10))
    per_window = [(stamps[warmup + (w + 1) * window] - stamps[warmup + w * window]) / window * 1e3 for w in range(steps // window)]
    return {"tok_s": batch * steps / seconds, "ms_per_step": seconds / steps * 1e3, "h2d_bytes": engine.runner.packer._cursor * 4,
            "d2h_bytes": batch * 4, "steps": steps, "ms_per_step_median": round(statistics.median(per_window), 4),
            "ms_per_step_p10": round(percentile(per_window, 0.1), 4), "ms_per_step_p90": round(percentile(per_window, 0.9), 4)}


def other_workload(name: str) -> int:
    """The two larger workloads: continuous batching through ``Engine.generate`` with host tokens in and out."""
    import torch

    from hyperion_b200.api import Engine
    from hyperion_b200.config import Qwen2Config
    from hyperion_b200.sampling import SamplingParams

    if name == "mixed-1.5b":
        config = Qwen2Config(num_hidden_layers=28, hidden_size=1536, intermediate_size=8960, num_attention_heads=12, num_key_value_heads=2,
                             head_dim=128, vocab_size=151936, max_position_embeddings=32768, rope_theta=1e6, rms_norm_eps=1e-6,
                             tie_word_embeddings=True)
        lengths = torch.randint(16, 4097, (128,), generator=torch.Generator().manual_seed(0)).tolist()
        new_tokens, max_batch, budget = 256, 128, 8192
    else:
        config = Qwen2Config(num_hidden_layers=64, hidden_size=5120, intermediate_size=27648, num_attention_heads=40, num_key_value_heads=8,
                             head_dim=128, vocab_size=152064, max_position_embeddings=32768, rope_theta=1e6, rms_norm_eps=1e-6,
                             tie_word_embeddings=False)
        lengths = [4096] * 16
        new_tokens, max_batch, budget = 512, 16, 8192
    prompts = [random_prompt(i, n, config.vocab_size) for i, n in enumerate(lengths)]
    cache_tokens = sum(-(-(n + new_tokens) // 16) * 16 for n in lengths)
    engine = Engine.from_random("Qwen2ForCausalLM", config, seed=0, dtype="bfloat16", page_size=16, max_tokens=cache_tokens, max_requests=max_batch)
    params = SamplingParams(temperature=0.0, max_tokens=new_tokens, ignore_eos=True)
    engine.generate(prompts[:2], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))  # warm-up: compiles, library set-up
    torch.cuda.synchronize()
    started = time.perf_counter()
    outputs = engine.generate(prompts, params, max_batch=max_batch, max_batch_tokens=budget, prefill_chunk_busy=2048)
    seconds = time.perf_counter() - started
    generated, prompt_tokens = sum(len(o) for o in outputs), sum(lengths)
    print(json.dumps({"workload": name, "requests": len(prompts), "prompt_tokens": prompt_tokens, "generated_tokens": generated,
                      "seconds": round(seconds, 3), "generated_tokens_per_s": round(generated / seconds, 1),
                      "all_tokens_per_s": round((generated + prompt_tokens) / seconds, 1), "steps": engine.runner.steps_run,
                      "graphs": len(engine.runner.graphs), "dtype": "bf16", "data": "synthetic: random weights and token ids",
                      "layers": config.num_hidden_layers, "hidden": config.hidden_size}))
    return 0


def reference_tables() -> int:
    """The reference's own published tables at their shapes (docs/performance-log.md:369-384,197,243-244,407, measured on an
    H100): decode ms per step by batch at context 512 and prefill ms by prompt length, for the 0.5B and the 7B shape."""
    import torch

    from hyperion_b200.api import Engine
    from hyperion_b200.config import Qwen2Config
    from hyperion_b200.engine.batch import StepEntry
    from hyperion_b200.sampling import GREEDY, pack_options

    shapes = {
        "0.5b": (Qwen2Config(num_hidden_layers=24, hidden_size=896, intermediate_size=4864, num_attention_heads=14, num_key_value_heads=2, head_dim=64,
                             vocab_size=151936, max_position_embeddings=32768, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True),
                 {"decode_ms_h100": {1: 1.502, 2: 1.747, 4: 1.771, 8: 1.806, 16: 1.918, 32: 2.219}, "prefill_ms_h100": {1024: 6.2, 4096: 23.3, 8192: 59.4, 16384: 175.5}}),
        "7b": (model_config(28),
               {"decode_ms_h100": {1: 6.763, 2: 6.780, 4: 6.826, 8: 7.263, 16: 7.793, 32: 8.855}, "prefill_ms_h100": {1024: 32.85, 4096: 146.36, 8192: 343.29, 16384: 916.06}}),
    }
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, (config, published) in shapes.items():
        engine = Engine.from_random("Qwen2ForCausalLM", config, seed=0, dtype="bfloat16", page_size=16, max_tokens=32 * 640 + 17000, max_requests=32)
        vocab = config.vocab_size
        prefill = {}
        for tokens in published["prefill_ms_h100"]:
            ids = random_prompt(tokens, tokens, vocab)
            times = []
            for rep in range(5):  # the first two run directly, the third is captured, the last two are replays
                torch.cuda.synchronize()
                start.record()
                engine.step([StepEntry(f"p{tokens}_{rep}", ids, [tokens - 1])])
                stop.record()
                torch.cuda.synchronize()
                times.append(start.elapsed_time(stop))
                engine.finish(f"p{tokens}_{rep}")
            prefill[tokens] = round(min(times[3:]), 3)
        decode = {}
        for batch in published["decode_ms_h100"]:
            names = [f"d{batch}_{i}" for i in range(batch)]
            for i, request in enumerate(names):
                engine.step([StepEntry(request, random_prompt(i, 512, vocab), [])])
            options = {"sampling_options": ([w for request in names for w in pack_options(GREEDY, 0, engine.cache.slot(request))], (batch, 8))}

            def one():
                logits = engine.runner.step([StepEntry(request, [5], [0]) for request in names], options)
                engine.sampler.sample(logits, engine.runner.last_context.extra["sampling_options"], all_greedy=True)

            for _ in range(5):
                one()
            torch.cuda.synchronize()
            start.record()
            for _ in range(32):
                one()
            stop.record()
            torch.cuda.synchronize()
            decode[batch] = round(start.elapsed_time(stop) / 32, 3)
            for request in names:
                engine.finish(request)
        engine.check()
        print(json.dumps({"workload": "reference-tables", "shape": name, "dtype": "bf16", "data": "synthetic: random weights and token ids",
                          "decode_ms_per_step_at_context_512": decode, "prefill_ms": prefill, "published_h100": published}))
        del engine
        torch.cuda.empty_cache()
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128, help="decode steps per timed window (at most a tenth of the range, so that there are ten windows)")
    parser.add_argument("--warmup", type=int, default=8, help="untimed decode steps before the first window (at least 3)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=28, help="fewer than the configuration's 28 only to save memory or time")
    parser.add_argument("--decode-tokens", type=int, default=CONTEXT - PROMPT,
                        help="tokens decoded after the 2,048-token prompts (the configuration's range is 2,048, to context 4,096); fewer only for profiling")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--skip-points", action="store_true", help="leave out the batch 1 / 64 points, prefill and e2e")
    parser.add_argument("--only", default=None, choices=["prefill"], help="time one part alone (for profiling)")
    parser.add_argument("--workload", default=None, choices=["mixed-1.5b", "batch-32b", "reference-tables"],
                        help="one of the other workloads instead: 128 requests with prompts of 16..4096 tokens and 256 decoded tokens "
                             "each through generate() at the 1.5B shape; batch 16 with prompts of 4,096 and 512 decoded tokens at the 32B shape; "
                             "or the reference's own published tables (decode by batch at context 512, prefill by length) at the 0.5B and 7B shapes")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.workload == "reference-tables":
        return reference_tables()
    if args.workload:
        return other_workload(args.workload)
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print("bench.py: this engine runs on one GPU; --gpus > 1 is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    args.steps = max(1, args.steps)
    decode_tokens = max(args.warmup + 10, min(args.decode_tokens, CONTEXT - PROMPT))

    import torch

    from hyperion_b200.api import Engine

    measured, source = peaks()
    config = model_config(args.layers)
    largest = args.batch if args.skip_points else max(args.batch, 64)
    tokens_needed = largest * (PROMPT + decode_tokens + 16) + PROMPT + 16
    engine = Engine.from_random("Qwen2ForCausalLM", config, seed=0, dtype="bfloat16", page_size=16,
                                max_tokens=tokens_needed, max_requests=max(largest, 8))
    if args.only == "prefill":  # for profiling: the prefill step alone
        prefill = time_prefill(engine, reps=max(1, args.steps), warmup=args.warmup)
        print(json.dumps({"only": "prefill", "layers": args.layers, "tokens": PROMPT, "ms": round(prefill["ms"], 3),
                          "tokens_per_s": round(PROMPT / (prefill["ms"] / 1e3), 1)}))
        return 0
    # The prompt step first, on a GPU that has been idle: a burst of eight 22 ms steps, set against the burst peak. Under
    # sustained load the board's power cap lowers the clocks within a few hundred milliseconds; that figure is taken at
    # the end, after the decode runs, and set against the sustained peak.
    prefill = None if args.skip_points else time_prefill(engine)
    clocks = ClockSampler()
    clocks.start()
    main_run = time_decode(engine, args.batch, args.steps, args.warmup, decode_tokens)
    clock_record = clocks.stop()

    def roofline(run: dict, batch: int) -> dict:
        bytes_per_step = weight_bytes(config) + batch * run["mean_context"] * engine.cache.bytes_per_token()
        achieved = bytes_per_step / (run["ms_per_step"] / 1e3) / 1e9
        return {"bound": "hbm", "achieved": round(achieved, 1), "peak": measured["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / measured["hbm_gbs"], 4), "of": source, "mean_context": round(run["mean_context"], 1)}

    record = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Qwen2.5-7B)",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": main_run["window"], "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        # the only published number there is: another GPU and a shorter context (see "baseline"), so a ratio across hardware
        "vs_baseline": round(main_run["tok_s"] / BASELINE_TOK_S[args.batch], 3) if args.batch in BASELINE_TOK_S else None,
        "baseline": {**BASELINE_LABEL, "value": BASELINE_TOK_S.get(args.batch)},
        "dtype": "bf16", "data": "synthetic: seeded random weights (N(0, 0.02)) and uniform random token ids",
        "impl": "ours",
        "config": {"model": "Qwen2.5-7B shape", "layers": args.layers, "layers_of_config": 28, "hidden": config.hidden_size,
                   "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
                   "intermediate": config.intermediate_size, "vocab": config.vocab_size, "global_batch": args.batch,
                   "seq_len": PROMPT + decode_tokens, "prompt_len": PROMPT, "decoded_tokens_per_request": decode_tokens,
                   "timed_steps": main_run["steps"], "page_size": 16, "parallelism": "single GPU",
                   "l2": "weights (15 GB) exceed L2; every step streams them", "peaks": source},
        "windows": main_run["windows"],
        "clocks": clock_record,
        "gpu_launches": main_run["launches"],
        "host_ms_per_step": round(main_run["host_ms_per_step"], 4),
        "roofline": roofline(main_run, args.batch),
    }
    if not args.skip_points:
        flops = prefill_flops(config, PROMPT)
        record["prefill"] = {"value": round(PROMPT / (prefill["ms"] / 1e3), 1), "tokens": PROMPT, "ms": round(prefill["ms"], 3),
                             "frac": round(flops / (prefill["ms"] / 1e3) / (measured["bf16_tflops"] * 1e12), 4), "of": source,
                             "regime": "burst: median of 5 replays after 3 warm-ups on an idle GPU, against the burst peak"}
        record["points"], record["points_detail"] = {}, {}
        for batch in (1, 64):
            run = time_decode(engine, batch, args.steps, args.warmup, decode_tokens)
            record["points"][f"decode_b{batch}"] = round(run["tok_s"], 1)
            record["points_detail"][f"decode_b{batch}"] = {"ms_per_step": round(run["ms_per_step"], 4), "timed_steps": run["steps"], "windows": run["windows"],
                                                           "roofline_frac": roofline(run, batch)["frac"]}
        sustained = time_prefill(engine, reps=20, warmup=10)  # the GPU has been under load for a while by now
        sustained_peak = measured.get("bf16_tflops_sustained", measured["bf16_tflops"])
        record["prefill"].update({"sustained_ms": round(sustained["ms"], 3), "sustained_value": round(PROMPT / (sustained["ms"] / 1e3), 1),
                                  "sustained_frac": round(flops / (sustained["ms"] / 1e3) / (sustained_peak * 1e12), 4)})
        e2e = time_e2e(engine, args.batch, args.steps, args.warmup, decode_tokens)
        record["e2e"] = {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d_bytes"],
                         "d2h_bytes_per_step": e2e["d2h_bytes"], "ms_per_step": round(e2e["ms_per_step"], 4), "timed_steps": e2e["steps"],
                         "ms_per_step_median": e2e["ms_per_step_median"], "ms_per_step_p10": e2e["ms_per_step_p10"],
                         "ms_per_step_p90": e2e["ms_per_step_p90"], "clock": "host"}
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
