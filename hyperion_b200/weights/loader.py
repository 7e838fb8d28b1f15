"""Loading a model's tensors from a folder of safetensors by name.

The names and shapes a model expects come from its parts.  A tensor that is missing, one that no
part asked for, and one with another shape are all errors, reported together in one message, as the
reference refuses missing, unmapped and mis-shaped tensors
(ignition/src/hyperion_ignition/compiler/weights.py:231-261).  Element types: in the bfloat16 mode a
tensor stored in 16 bits is kept as bfloat16 and a tensor stored in 32 bits stays float32; in the
float32 mode every floating tensor becomes float32 (bfloat16 widens exactly); integer tables become
int32.
"""
from __future__ import annotations

from pathlib import Path
from typing import Mapping

import torch

from ..parts.base import WeightSpec
from .safetensors_io import TensorEntry, TensorFiles, read_model_index


class WeightsError(ValueError):
    """The folder's tensors do not match what the model expects."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_type):
        lines = []
        if missing:
            lines.append(f"missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"wrong shapes ({len(wrong_shape)}): " + ", ".join(f"{n} is {list(f)}, expected {list(e)}" for n, f, e in wrong_shape))
        if wrong_type:
            lines.append(f"wrong element types ({len(wrong_type)}): " + ", ".join(f"{n} is {t}" for n, t in wrong_type))
        super().__init__("the checkpoint does not match the model:\n  " + "\n  ".join(lines))
        self.missing, self.unexpected, self.wrong_shape, self.wrong_type = missing, unexpected, wrong_shape, wrong_type


def check_tensors(found: Mapping[str, TensorEntry], expected: Mapping[str, WeightSpec], tolerated=()) -> None:
    missing = sorted(set(expected) - set(found))
    unexpected = sorted(set(found) - set(expected) - set(tolerated))
    wrong_shape, wrong_type = [], []
    for name in sorted(set(found) & set(expected)):
        entry, wanted = found[name], expected[name]
        if tuple(entry.shape) != tuple(wanted.shape):
            wrong_shape.append((name, entry.shape, wanted.shape))
        if wanted.integer == entry.dtype.is_floating_point:
            wrong_type.append((name, str(entry.dtype)))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightsError(missing, unexpected, wrong_shape, wrong_type)


def stored_to_runtime(tensor: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if not tensor.is_floating_point():
        return tensor.to(torch.int32)
    if dtype == torch.float32 or tensor.dtype in (torch.float32, torch.float64):
        return tensor.to(torch.float32)
    return tensor.to(torch.bfloat16)


def load_weights(model, model_dir: Path, progress=None) -> None:
    """Read the folder, check it against ``model.expected_tensors()`` and hand the tensors to the parts."""
    found = read_model_index(Path(model_dir))
    expected = model.expected_tensors()
    check_tensors(found, expected, model.spec.tolerated)
    files = TensorFiles()
    tensors = {}
    try:
        for count, name in enumerate(expected):
            tensors[name] = stored_to_runtime(files.read(found[name]), model.dtype).to(model.device)
            if progress is not None:
                progress(count + 1, len(expected))
    finally:
        files.close()
    model.load(tensors)
