"""Sampling options of a request, with the reference's names, defaults and ranges.

``temperature`` 0 is greedy (argmax of the raw logits); ``top_k`` 0 keeps the whole vocabulary;
``repetition_penalty`` divides positive and multiplies negative logits of tokens the request has
generated (the prompt does not count) and is refused together with temperature 0; an absent
``seed`` is drawn from the operating system and reported
(helios/crates/helios-core/src/api.rs:111-189; helios/crates/helios-hal/src/sampler_reference.rs:4-26).
``max_tokens`` bounds the generated tokens (default 1024, api.rs:193); ``ignore_eos`` keeps
generating past an end-of-sequence token, for benchmarks that decode a fixed count.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, replace
from typing import Optional

DEFAULT_MAX_TOKENS = 1024


class InvalidParameter(ValueError):
    def __init__(self, name: str, reason: str):
        super().__init__(f"{name} {reason}")
        self.name = name


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    repetition_penalty: float = 1.0
    seed: Optional[int] = None
    max_tokens: int = DEFAULT_MAX_TOKENS
    ignore_eos: bool = False

    def validated(self) -> "SamplingParams":
        if not (isinstance(self.temperature, (int, float)) and 0.0 <= self.temperature <= 2.0):
            raise InvalidParameter("temperature", "must be between 0 and 2")
        if not (isinstance(self.top_p, (int, float)) and 0.0 <= self.top_p <= 1.0):
            raise InvalidParameter("top_p", "must be between 0 and 1")
        if isinstance(self.top_k, bool) or not isinstance(self.top_k, int) or self.top_k < 0:
            raise InvalidParameter("top_k", "must be a non-negative integer")
        if not (isinstance(self.repetition_penalty, (int, float)) and self.repetition_penalty > 0 and math.isfinite(self.repetition_penalty)):
            raise InvalidParameter("repetition_penalty", "must be positive")
        if self.temperature == 0 and self.repetition_penalty != 1.0:
            raise InvalidParameter("repetition_penalty", "is not supported with temperature 0 (greedy decoding)")
        if isinstance(self.max_tokens, bool) or not isinstance(self.max_tokens, int) or not 0 < self.max_tokens < 1 << 31:
            raise InvalidParameter("max_tokens", "must be a positive integer below 2^31")
        seed = self.seed
        if seed is None:
            seed = int.from_bytes(os.urandom(8), "little")
        if isinstance(seed, bool) or not isinstance(seed, int) or not 0 <= seed < 1 << 64:
            raise InvalidParameter("seed", "must be an unsigned 64-bit integer")
        return replace(self, seed=seed, temperature=float(self.temperature), top_p=float(self.top_p),
                       repetition_penalty=float(self.repetition_penalty))

    @property
    def greedy(self) -> bool:
        return self.temperature == 0


GREEDY = SamplingParams(temperature=0.0)
