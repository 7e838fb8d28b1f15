"""The sampler: a device kernel that picks one token per row of logits, and a slow host reference of
the same rule for tests.

The rule follows the reference's steps (helios/crates/helios-hal/src/sampler_reference.rs:4-26):
penalty on generated tokens, division by the temperature, the top-k set (value descending, ties
to the lower index), the nucleus over that set (smallest prefix whose mass reaches top_p of the
set's mass), then one uniform draw ``u`` from Philox4x32-10 with key = the request's seed and
counter = the number of tokens it sampled before.  One step differs: the token is the first,
walking the kept tokens by **ascending index**, at which the running mass exceeds ``u`` times the
kept mass; the reference walks them in its sorted order (value descending) with float32 prefix sums
in segments of 1,024 (sampler_reference.rs steps 5-7).  The kept set, every token's probability and
therefore the distribution are the same; a given seed and step may pick another token than the
reference would.  Walking by index needs no sort of the kept set on the device.
"""
from __future__ import annotations

import struct
from typing import Optional, Sequence

import numpy as np
import torch

from ..ops.native import check, i32, library, ptr, require_cuda, stream_ptr
from .params import SamplingParams

MASK32 = 0xFFFFFFFF


def philox4x32_10(counter: Sequence[int], key: Sequence[int]) -> list[int]:
    """Philox4x32 with 10 rounds (Salmon et al., SC11), as the reference uses it
    (helios/crates/helios-hal/src/sampler_reference.rs:67-84)."""
    c, k = list(counter), list(key)
    for round_index in range(10):
        p0, p1 = 0xD2511F53 * c[0], 0xCD9E8D57 * c[2]
        c = [(p1 >> 32) ^ c[1] ^ k[0], p1 & MASK32, (p0 >> 32) ^ c[3] ^ k[1], p0 & MASK32]
        if round_index < 9:
            k = [(k[0] + 0x9E3779B9) & MASK32, (k[1] + 0xBB67AE85) & MASK32]
    return c


def uniform(seed: int, step: int) -> float:
    """The draw in [0, 1) of a request's ``step``-th sampled token (sampler_reference.rs:87-90)."""
    word = philox4x32_10([step & MASK32, 0, 0, 0], [seed & MASK32, (seed >> 32) & MASK32])[0]
    return (word >> 8) / 16777216.0


def reference_sample(logits: np.ndarray, params: SamplingParams, step: int, generated: Sequence[int] = ()) -> tuple[int, dict]:
    """The token the rule picks, computed in float64 with a sort; also the interval of ``u`` values
    that pick it and the kept set, so a test can accept a device result that differs only because
    ``u`` fell within rounding of a boundary."""
    z = np.asarray(logits, dtype=np.float64).copy()
    z[np.isnan(z)] = -np.inf
    if params.temperature == 0:
        return int(np.argmax(z)), {}
    if params.repetition_penalty != 1.0:
        for token in set(generated):
            z[token] = z[token] / params.repetition_penalty if z[token] > 0 else z[token] * params.repetition_penalty
    z = z.astype(np.float32).astype(np.float64) / np.float64(np.float32(params.temperature))
    order = np.lexsort((np.arange(z.size), -z))  # value descending, ties by lower index
    kk = z.size if params.top_k == 0 else min(params.top_k, z.size)
    kept = order[:kk]
    weights = np.exp(z[kept] - z.max())
    if params.top_p < 1.0:
        cumulative = np.cumsum(weights)
        need = np.float64(np.float32(params.top_p)) * cumulative[-1]
        keep = int(np.searchsorted(cumulative, need, side="left")) + 1
        kept, weights = kept[:keep], weights[:keep]
    by_index = np.argsort(kept)
    kept, weights = kept[by_index], weights[by_index]
    running = np.cumsum(weights)
    u = uniform(params.seed, step)
    target = u * running[-1]
    j = int(np.searchsorted(running, target, side="right"))
    j = min(j, kept.size - 1)
    lower = (running[j - 1] if j else 0.0) / running[-1]
    return int(kept[j]), {"u": u, "interval": (lower, running[j] / running[-1]), "kept": kept, "cdf": running / running[-1]}


def _float_bits(value: float) -> int:
    return struct.unpack("<i", struct.pack("<f", value))[0]


def _signed(word: int) -> int:
    return word - (1 << 32) if word >= 1 << 31 else word


def pack_options(params: SamplingParams, step: int, slot: int) -> list[int]:
    """The 8 int32 words the kernel reads for one row."""
    seed = params.seed or 0
    return [_float_bits(params.temperature), _float_bits(params.top_p), _float_bits(params.repetition_penalty), int(params.top_k),
            _signed(seed & MASK32), _signed((seed >> 32) & MASK32), _signed(step & MASK32), int(slot)]


class Sampler:
    """Launches the sampling kernel.  ``seen`` is the per-request bitmap of generated tokens
    ([slots, ceil(vocab / 32)] int32, a fixed-size state record of the cache manager)."""

    def __init__(self, vocab: int, device: torch.device, seen: Optional[torch.Tensor] = None):
        self.vocab = vocab
        self.device = device
        self.seen = seen

    @staticmethod
    def seen_words(vocab: int) -> int:
        return (vocab + 31) // 32

    ARGMAX_CHUNKS = 32

    def sample(self, logits: torch.Tensor, options: torch.Tensor, out: Optional[torch.Tensor] = None, all_greedy: bool = False) -> torch.Tensor:
        """``logits`` [rows, vocab] float32; ``options`` [rows, 8] int32 on the device (see ``pack_options``).
        ``all_greedy``: the caller knows every row has temperature 0; the argmax then runs spread over many blocks
        per row instead of one."""
        require_cuda(logits, options)
        rows = logits.shape[0]
        if logits.dtype != torch.float32 or logits.stride(-1) != 1 or logits.shape[1] != self.vocab:
            raise ValueError("sampler: logits must be float32 [rows, vocab]")
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        seen_words = self.seen.shape[-1] if self.seen is not None else 0
        if all_greedy:
            chunks = self.ARGMAX_CHUNKS
            workspace = torch.empty(2 * rows * chunks, dtype=torch.int32, device=logits.device)
            check(library("sampling").hb_argmax(ptr(logits), i32(logits.stride(0)), i32(rows), i32(self.vocab), i32(chunks), ptr(workspace),
                                                ptr(options), ptr(self.seen), i32(seen_words), ptr(out), stream_ptr()), "argmax")
            return out
        check(library("sampling").hb_sample(ptr(logits), i32(logits.stride(0)), i32(rows), i32(self.vocab), ptr(options), ptr(self.seen),
                                 i32(seen_words), ptr(out), stream_ptr()), "sample")
        return out
