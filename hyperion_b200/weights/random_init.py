"""Seeded random weights: in memory for a model, or written out as a model folder.

The reference has no random-weight mode; its tiny fixture is a saved default initialisation
(scripts/gen-sharded-fixture.py:32-50).  Here every tensor is a pure function of the seed, its own
name and the element's index (``philox_normal``): matrices and biases N(0, std), norm weights
1 + N(0, std), rounded to bfloat16.  The device fills a tensor with a kernel and the host with numpy,
and both give the same bits, so ``Engine.from_random(seed)`` holds the very model that
``write_model_folder(seed)`` writes, and a tensor's values do not depend on which other tensors exist.
"""
from __future__ import annotations

import ctypes
import json
from pathlib import Path
from typing import Any

import torch

from ..parts.base import WeightSpec
from . import philox_normal
from .safetensors_io import write_file


def random_tensor(name: str, wanted: WeightSpec, seed: int, std: float, device: torch.device, dtype: torch.dtype) -> torch.Tensor:
    """The tensor ``name`` of the model with this seed, made where it is wanted: by the kernel of ``csrc/random_normal.cu``
    on a CUDA device, by numpy elsewhere; the values are the same."""
    device = torch.device(device)
    if wanted.integer:
        return torch.zeros(wanted.shape, dtype=torch.int32, device=device)
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"random weights are made as bfloat16 or float32, got {dtype}")
    key = philox_normal.tensor_key(seed, name)
    mean = 1.0 if wanted.init == "one_plus_normal" else 0.0
    count = 1
    for extent in wanted.shape:
        count *= int(extent)
    if device.type == "cuda":
        from ..ops.native import check, library, ptr, stream_ptr

        out = torch.empty(wanted.shape, dtype=dtype, device=device)
        constants = philox_normal.constants()
        with torch.cuda.device(device):
            check(library("random_normal").hb_random_normal(ptr(out), int(dtype == torch.bfloat16), ctypes.c_longlong(count), ctypes.c_uint(key[0]),
                                                            ctypes.c_uint(key[1]), ctypes.c_double(std), ctypes.c_double(mean), ctypes.byref(constants),
                                                            stream_ptr()), "random_normal")
        return out
    values = torch.from_numpy(philox_normal.normal_float32(count, key, std, mean))
    return values.to(dtype).view(wanted.shape).to(device)


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
                       stored: torch.dtype = torch.bfloat16, device=None) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with weights from ``seed``.  ``device``: where the
    values are made (a CUDA device when one is visible, else the host); the file is the same either way."""
    from ..models import DecoderModel, get_architecture

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    entry = get_architecture(architecture)
    model = DecoderModel(entry.build_spec(config), torch.float32, torch.device("meta"))
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    tensors = {name: tensor.cpu() for name, tensor in random_tensors(model, seed, std, stored, device=torch.device(device)).items()}
    with open(folder / "config.json", "w", encoding="utf-8") as handle:
        json.dump(entry.write_config(config), handle, indent=1)
    write_file(folder / "model.safetensors", tensors)
    return folder
