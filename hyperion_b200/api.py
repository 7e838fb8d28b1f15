"""The Python entry point: load a model folder (or random weights) and step or generate with it.

``Engine`` owns the model, the cache manager and the step function; ``generate`` drives them with
the scheduler and the sampler.  The reference's nearest calls are the backend's load order
``load_model -> reserve_kv -> commit_kv -> submit_step`` (helios/crates/helios-hal/src/traits.rs:69-121)
and its direct ``generate`` (helios/crates/helios-hal/src/backends/hopper_sm90/forward_device.rs:50-60).
"""
from __future__ import annotations

from collections import deque
from pathlib import Path
from typing import Any, Optional, Sequence

import numpy as np
import torch

from . import host as host_runtime
from .cache.manager import CacheManager, OutOfPages
from .config.generation import GenerationDefaults, read_generation_defaults
from .engine.batch import BadStep, StepEntry
from .engine.runner import ModelRunner
from .models import DecoderModel, get_architecture, read_model_config
from .parts.base import RequestState
from .sampling import Sampler, SamplingParams, pack_options
from .weights import init_random, load_weights

SAMPLER_STATE = -1  # the cache manager's user id of the sampler's per-request record

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    if dtype not in DTYPES:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {dtype!r}")
    return DTYPES[dtype]


class Engine:
    """A loaded model with its cache.

    ``page_size`` tokens per cache page (a power of two); the cache holds ``max_tokens`` tokens in
    every group of layers (rounded up to whole pages); at most ``max_requests`` requests are live.
    """

    def __init__(self, model: DecoderModel, config: Any, page_size: int = 16, max_tokens: int = 4096, max_requests: int = 64,
                 defaults: Optional[GenerationDefaults] = None):
        self.model = model
        self.config = config
        self.dtype = model.dtype
        self.device = model.device
        self.page_size = page_size
        self.defaults = defaults or GenerationDefaults(eos_token_ids=tuple(getattr(config, "eos_token_ids", ()) or ()))
        num_pages = max(1, -(-max_tokens // page_size))
        vocab = model.spec.vocab_size
        users = model.cache_users() + [(SAMPLER_STATE, RequestState((Sampler.seen_words(vocab),), torch.int32))]
        self.cache = CacheManager(users, page_size, num_pages, max_requests, dtype=model.dtype, device=model.device)
        self.runner = ModelRunner(model, self.cache)
        self.sampler = Sampler(vocab, model.device, seen=self.cache.state_storage(SAMPLER_STATE))
        self._token_staging = torch.empty((2, max(1, max_requests)), dtype=torch.int32, pin_memory=True)
        self._token_ring = torch.empty((2, max(1, max_requests)), dtype=torch.int32, device=model.device)

    # ------------------------------------------------------------------ construction
    @staticmethod
    def _device(device) -> torch.device:
        if not torch.cuda.is_available():
            raise RuntimeError("hyperion_b200 needs a CUDA device (sm_100a); none is visible and there is no CPU path")
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError(f"hyperion_b200 runs on CUDA devices only, got {device}")
        torch.cuda.set_device(device)
        return torch.device("cuda", torch.cuda.current_device())

    @classmethod
    def from_folder(cls, model_dir, dtype="bfloat16", device="cuda:0", **cache_options) -> "Engine":
        """Load ``config.json`` and the safetensors of ``model_dir``; the model class comes from config.json."""
        model_dir = Path(model_dir)
        architecture, config = read_model_config(model_dir)
        model = DecoderModel(architecture.build_spec(config), resolve_dtype(dtype), cls._device(device))
        load_weights(model, model_dir)
        return cls(model, config, defaults=read_generation_defaults(model_dir), **cache_options)

    @classmethod
    def from_random(cls, architecture: str, config: Any, seed: int = 0, std: float = 0.02, dtype="bfloat16", device="cuda:0",
                    **cache_options) -> "Engine":
        """A model of ``config`` with seeded random weights made on the device (no files)."""
        entry = get_architecture(architecture)
        model = DecoderModel(entry.build_spec(config), resolve_dtype(dtype), cls._device(device))
        init_random(model, seed, std)
        return cls(model, config, **cache_options)

    # ------------------------------------------------------------------ stepping
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """See :meth:`hyperion_b200.engine.runner.ModelRunner.step`."""
        return self.runner.step(entries)

    def finish(self, request) -> None:
        self.runner.finish(request)

    # ------------------------------------------------------------------ generation
    def generate(self, prompts: Sequence[Sequence[int]], sampling=None, *, max_batch: Optional[int] = None,
                 max_batch_tokens: int = 2048, prefill_chunk_busy: int = 512, max_seq_len: Optional[int] = None,
                 on_token=None, return_reasons: bool = False, lookahead: bool = True):
        """Generate a continuation for every prompt (lists of token ids) with continuous batching.

        ``sampling`` is one :class:`SamplingParams` for all prompts or one per prompt; missing fields
        take the model folder's ``generation_config.json`` defaults.  Returns the generated ids per
        prompt (with ``return_reasons`` also why each ended: ``stop``, ``length`` or a failure text).
        ``on_token(index, token)`` is called as tokens appear; when it returns ``False`` that request is cancelled
        (its pages are freed at once, its reason is ``cancelled``; the reference's scheduler cancels the same way,
        helios/crates/helios-core/src/step_scheduler.rs:132-154).  With ``lookahead`` the next step is
        launched before the last one's ids have reached the host (it takes them on the device), so
        the device never waits for the host; ids then appear one step late, and a request that
        ends on an end-of-sequence token has run one row in vain.
        """
        from .engine.scheduler import Request, Scheduler, SchedulerConfig

        prompts = [list(p) for p in prompts]
        if sampling is None:
            d = self.defaults
            sampling = SamplingParams(temperature=d.temperature, top_p=d.top_p, top_k=d.top_k, repetition_penalty=d.repetition_penalty)
        per_prompt = list(sampling) if isinstance(sampling, (list, tuple)) else [sampling] * len(prompts)
        if len(per_prompt) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        limit = self.model.spec.max_positions
        if max_seq_len is not None:
            if not 0 < max_seq_len <= limit:
                raise ValueError(f"max_seq_len {max_seq_len} is outside 1..={limit} (the model's limit)")
            limit = max_seq_len
        scheduler = Scheduler(SchedulerConfig(
            num_pages=self.cache.num_pages, page_size=self.page_size, max_seq_len=limit,
            max_batch=min(max_batch or self.cache.max_requests, self.cache.max_requests), max_batch_tokens=max_batch_tokens,
            prefill_chunk_busy=prefill_chunk_busy, eos_token_ids=tuple(self.defaults.eos_token_ids), max_in_flight=2 if lookahead else 1,
            group_windows=tuple(self.cache.group_windows)))
        # Requests are known to the scheduler by keys 0..n-1 (their order here) and to the cache by keys of its own.
        per_prompt = [p.validated() for p in per_prompt]  # once: an absent seed is drawn here, for the scheduler's copy and the sampler's alike
        sched_keys = [scheduler.enqueue(Request(index, prompt, params)) for index, (prompt, params) in enumerate(zip(prompts, per_prompt))]
        assert sched_keys == list(range(len(prompts)))
        base_options = np.asarray([pack_options(p, 0, 0) for p in per_prompt], dtype=np.int32).reshape(len(prompts), 8)
        greedy = np.asarray([p.greedy for p in per_prompt], dtype=bool)
        cache_key = np.full(len(prompts), -1, dtype=np.int64)  # the cache's key of each request once it is live
        self._generate_calls = getattr(self, "_generate_calls", 0) + 1
        names = [("generate", self._generate_calls, index) for index in range(len(prompts))]  # in the cache: apart from a caller's own requests
        outputs: list[list[int]] = [[] for _ in prompts]
        reasons: list[Optional[str]] = [None] * len(prompts)

        def take_events():
            keys, kinds, tokens, texts = scheduler.take_event_arrays()
            for key, kind, token, text in zip(keys.tolist(), kinds.tolist(), tokens.tolist(), texts):
                if kind == 0:
                    outputs[key].append(token)
                    if on_token is not None and on_token(key, token) is False:
                        scheduler.cancel(key)  # the caller wants no more of this request: it ends with reason "cancelled"
                else:
                    reasons[key] = text

        def free_released():
            for key in scheduler.take_released_keys().tolist():
                if cache_key[key] >= 0 and self.cache.has(names[key]):
                    self.cache.free(names[key])
                cache_key[key] = -1

        depth = 2 if lookahead else 1
        in_flight: deque = deque()  # (plan, pinned ids or None, event), oldest first
        newest: Optional[tuple[int, torch.Tensor]] = None  # (plan step, its sampled ids on the device)
        launched = 0  # plans whose ids went into a ring slot: a plan that failed at launch takes none, whatever its step number

        def launch(plan):
            nonlocal newest, launched
            for key in plan.keys[cache_key[plan.keys] < 0].tolist():  # first portion of a prompt: the request becomes live
                self.cache.add_request(names[key])
                cache_key[key] = self.cache.keys.known(names[key])
            tokens, places = plan.tokens, None
            pending = np.flatnonzero(plan.from_step >= 0)
            if len(pending):  # sampled by the plan before, still on the device
                if newest is None or np.any(plan.from_step[pending] != newest[0]):
                    raise RuntimeError(f"plan {plan.step} wants tokens of a plan that is not the one before it")
                starts = np.cumsum(plan.counts) - plan.counts
                tokens = tokens.copy()
                tokens[starts[pending]] = 0
                places = dict(zip(pending.tolist(), plan.from_index[pending].tolist()))
            sampled_rows = np.flatnonzero(plan.sample)
            want = (np.cumsum(plan.counts)[sampled_rows] - 1).astype(np.int32)
            extra = None
            if len(sampled_rows):
                options = base_options[plan.keys[sampled_rows]]
                options[:, 6] = plan.sampled_before[sampled_rows]
                slots = np.empty(len(plan.keys), np.int32)
                lengths = np.empty(len(plan.keys), np.int32)
                keys = np.ascontiguousarray(cache_key[plan.keys])
                host_runtime.check(host_runtime.library().hb_cache_lengths(self.cache.native, len(keys), host_runtime.address(keys),
                                                                           host_runtime.address(lengths), host_runtime.address(slots)))
                options[:, 7] = slots[sampled_rows]
                extra = {"sampling_options": (options, (len(sampled_rows), 8))}
            logits = self.runner.step_arrays([names[key] for key in plan.keys.tolist()], np.ascontiguousarray(cache_key[plan.keys]), plan.counts, tokens, want, extra,
                                             device_tokens=(newest[1], places) if places else None)
            if logits is None:
                return plan, None, None
            # the slot of the plan `depth` launches ago, which has been retired: at most `depth` plans are in flight, oldest first
            ring = launched % depth
            launched += 1
            chosen = self.sampler.sample(logits, self.runner.last_context.extra["sampling_options"],
                                         out=self._token_ring[ring, : len(sampled_rows)], all_greedy=bool(greedy[plan.keys[sampled_rows]].all()))
            newest = (plan.step, chosen)
            pinned = self._token_staging[ring, : len(sampled_rows)]
            pinned.copy_(chosen, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
            return plan, pinned, event

        def retire(plan, pinned, event):
            if event is not None:
                event.synchronize()
            scheduler.complete_arrays(plan.step, pinned.numpy() if pinned is not None else np.empty(0, np.int32))
            take_events()
            free_released()

        try:
            while True:
                plan = scheduler.next_plan_arrays() if len(in_flight) < depth else None
                take_events()
                if plan is not None:
                    try:
                        in_flight.append(launch(plan))
                    except Exception as error:  # the step's requests fail, the others go on
                        scheduler.fail_step(plan.step, f"{type(error).__name__}: {error}")
                        take_events()
                        free_released()
                        if not isinstance(error, (OutOfPages, BadStep)):
                            raise
                        continue
                if in_flight and (plan is None or len(in_flight) >= depth):
                    retire(*in_flight.popleft())
                elif plan is None:
                    if scheduler.idle:
                        break
                    raise RuntimeError("the scheduler has requests but plans nothing")
        finally:  # whatever ended the loop, this call's requests leave the cache
            for key in np.flatnonzero(cache_key >= 0).tolist():
                if self.cache.has(names[key]):
                    self.cache.free(names[key])
        self.check()
        return (outputs, reasons) if return_reasons else outputs

    def check(self) -> None:
        """Wait for the device and raise if a kernel flagged a problem."""
        self.runner.check_device_status()
