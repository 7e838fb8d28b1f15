"""Seeded random weights: in memory for a model, or written out as a model folder.

The reference has no random-weight mode; its tiny fixture is a saved default initialisation
(scripts/gen-sharded-fixture.py:32-50).  Here every tensor is drawn from its own generator, seeded
from the seed and the tensor's name, so a tensor's values do not depend on which other tensors
exist: matrices and biases N(0, std), norm weights 1 + N(0, std), rounded to bfloat16.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any

import torch

from ..parts.base import WeightSpec
from .safetensors_io import write_file


def _tensor_seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:7], "little")


def random_tensor(name: str, wanted: WeightSpec, seed: int, std: float, device: torch.device, dtype: torch.dtype) -> torch.Tensor:
    generator = torch.Generator(device=device)
    generator.manual_seed(_tensor_seed(seed, name))
    if wanted.integer:
        return torch.zeros(wanted.shape, dtype=torch.int32, device=device)
    # drawn in chunks so that a 1e9-element matrix never holds a float32 copy of itself
    out = torch.empty(wanted.shape, dtype=dtype, device=device)
    flat = out.view(-1)
    chunk = 1 << 26
    for start in range(0, flat.numel(), chunk):
        part = torch.randn(min(chunk, flat.numel() - start), generator=generator, device=device, dtype=torch.float32) * std
        if wanted.init == "one_plus_normal":
            part += 1.0
        flat[start : start + part.numel()] = part.to(dtype)
    return out


def random_tensors(model, seed: int, std: float = 0.02, stored: torch.dtype = torch.bfloat16, device=None) -> dict[str, torch.Tensor]:
    """One tensor per name the model expects, with bfloat16-representable values (``stored``)."""
    device = torch.device(device) if device is not None else model.device
    return {name: random_tensor(name, wanted, seed, std, device, stored) for name, wanted in model.expected_tensors().items()}


def init_random(model, seed: int, std: float = 0.02) -> None:
    """Fill a model with random weights directly on its device (no files): bfloat16 values, widened
    exactly when the model runs in float32."""
    from .loader import stored_to_runtime

    tensors = {}
    for name, wanted in model.expected_tensors().items():
        tensors[name] = stored_to_runtime(random_tensor(name, wanted, seed, std, model.device, torch.bfloat16), model.dtype)
    model.load(tensors)


def write_model_folder(folder: Path, architecture: str, config: Any, seed: int, std: float = 0.02,
                       stored: torch.dtype = torch.bfloat16) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with weights from ``seed``."""
    from ..models import DecoderModel, get_architecture

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    entry = get_architecture(architecture)
    model = DecoderModel(entry.build_spec(config), torch.float32, torch.device("meta"))
    tensors = random_tensors(model, seed, std, stored, device=torch.device("cpu"))
    with open(folder / "config.json", "w", encoding="utf-8") as handle:
        json.dump(entry.write_config(config), handle, indent=1)
    write_file(folder / "model.safetensors", tensors)
    return folder
