"""End-of-sequence ids and sampling defaults of a model folder.

The end-of-sequence ids are the union of ``config.json`` and ``generation_config.json`` in that
order, and the sampling defaults (``temperature``, ``top_p``, ``top_k``, ``repetition_penalty``) are
whatever ``generation_config.json`` states, as in the reference
(ignition/src/hyperion_ignition/compiler/generation.py:51-71).  Unlike the reference, a folder
without any end-of-sequence id is accepted: random-weight folders have none and generation then
ends on its token limit.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any

from .base import ConfigError, ConfigReader, read_json

SAMPLING_KEYS = ("temperature", "top_p", "top_k", "repetition_penalty")


@dataclass(frozen=True)
class GenerationDefaults:
    eos_token_ids: tuple[int, ...] = ()
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    repetition_penalty: float = 1.0


def read_generation_defaults(model_dir: Path) -> GenerationDefaults:
    model_dir = Path(model_dir)
    eos: list[int] = []
    config = read_json(model_dir / "config.json")
    generation_path = model_dir / "generation_config.json"
    generation: dict[str, Any] = read_json(generation_path) if generation_path.is_file() else {}
    for document in (config, generation):
        for token in ConfigReader(document).token_ids("eos_token_id"):
            if token not in eos:
                eos.append(token)
    values: dict[str, Any] = {}
    for key in SAMPLING_KEYS:
        value = generation.get(key)
        if value is None:
            continue
        if isinstance(value, bool) or not isinstance(value, (int, float)) or value < 0:
            raise ConfigError(key, f"in generation_config.json must be a non-negative number, got {value!r}")
        values[key] = int(value) if key == "top_k" else float(value)
    return GenerationDefaults(eos_token_ids=tuple(eos), **values)
