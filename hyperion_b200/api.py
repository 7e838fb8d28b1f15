"""The Python entry point: load a model folder (or random weights) and step or generate with it.

``Engine`` owns the model, the cache manager and the step function; ``generate`` drives them with
the scheduler and the sampler.  The reference's nearest calls are the backend's load order
``load_model -> reserve_kv -> commit_kv -> submit_step`` (helios/crates/helios-hal/src/traits.rs:69-121)
and its direct ``generate`` (helios/crates/helios-hal/src/backends/hopper_sm90/forward_device.rs:50-60).
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Optional, Sequence

import torch

from .cache.manager import CacheManager
from .config.generation import GenerationDefaults, read_generation_defaults
from .engine.batch import StepEntry
from .engine.runner import ModelRunner
from .models import DecoderModel, get_architecture, read_model_config
from .weights import init_random, load_weights

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
        self.cache = CacheManager(model.cache_users(), page_size, num_pages, max_requests, dtype=model.dtype, device=model.device)
        self.runner = ModelRunner(model, self.cache)

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

    def check(self) -> None:
        """Wait for the device and raise if a kernel flagged a problem."""
        self.runner.check_device_status()
