"""Reading and writing the safetensors container without any helper library.  The header is parsed
and checked by the C++ host runtime; this module maps the files and hands out tensors.

Layout: an 8-byte little-endian header length, a JSON header ``{name: {dtype, shape,
data_offsets}}`` (``__metadata__`` is ignored) and the payload; a tensor starts at
``8 + header_len + begin`` (helios/crates/helios-hal/src/weights_plan.rs:38-46).  The checks follow
the reference's header reader (ignition/src/hyperion_ignition/compiler/weights.py:45-79): the header
must fit the file and stay under 64 MiB, every range must lie inside the payload, ``end - begin``
must equal the element count times the element size, ranges must not overlap, and no name may
come twice.  A model folder
holds either ``model.safetensors`` or a ``model.safetensors.index.json`` whose ``weight_map`` names
bare shard files (weights.py:127-174); both at once is an error.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable

import torch

_DTYPES: dict[str, torch.dtype] = {
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "F32": torch.float32,
    "F64": torch.float64,
    "I8": torch.int8,
    "U8": torch.uint8,
    "I16": torch.int16,
    "I32": torch.int32,
    "I64": torch.int64,
    "BOOL": torch.bool,
}
_NAMES = {dtype: name for name, dtype in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int  # offset inside the payload
    end: int
    path: Path
    payload_start: int  # 8 + header length


def _numel(shape: Iterable[int]) -> int:
    n = 1
    for extent in shape:
        n *= extent
    return n


def read_header(path: Path) -> dict[str, TensorEntry]:
    """The tensors one file declares, read and checked against the file's size by the host runtime
    (``csrc/host/safetensors.cpp``)."""
    from .. import host as host_runtime

    path = Path(path)
    if not path.is_file():
        raise FileNotFoundError(f"{path}: no such file")

    class _Refused(Exception):
        pass

    try:
        payload_start, found = host_runtime.safetensors_header(str(path), _Refused)
    except _Refused as refused:
        raise SafetensorsError(f"{path.name}: {refused}") from None
    return {name: TensorEntry(name, _DTYPES[dtype], shape, begin, end, path, payload_start) for name, dtype, shape, begin, end in found}


def read_model_index(model_dir: Path) -> dict[str, TensorEntry]:
    """Every tensor of a model folder, from the single file or from the shards its index names."""
    model_dir = Path(model_dir)
    single = model_dir / "model.safetensors"
    index = model_dir / "model.safetensors.index.json"
    if single.is_file() and index.is_file():
        raise SafetensorsError(f"{model_dir}: holds both model.safetensors and model.safetensors.index.json")
    if single.is_file():
        return read_header(single)
    if not index.is_file():
        raise FileNotFoundError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")
    with open(index, "r", encoding="utf-8") as handle:
        weight_map = json.load(handle).get("weight_map")
    if not isinstance(weight_map, dict) or not weight_map:
        raise SafetensorsError(f"{index.name}: no weight_map")
    by_shard: dict[str, set[str]] = {}
    for name, shard in weight_map.items():
        if not isinstance(shard, str) or Path(shard).name != shard:
            raise SafetensorsError(f"{index.name}: shard of {name!r} must be a bare file name, got {shard!r}")
        by_shard.setdefault(shard, set()).add(name)
    entries: dict[str, TensorEntry] = {}
    for shard, names in sorted(by_shard.items()):
        found = read_header(model_dir / shard)
        if set(found) != names:
            raise SafetensorsError(
                f"{shard}: holds {sorted(set(found) - names)} beyond the index and lacks {sorted(names - set(found))}"
            )
        entries.update(found)
    return entries


class TensorFiles:
    """Memory maps of the files behind a set of entries; tensors are read out as copies."""

    def __init__(self) -> None:
        self._maps: dict[Path, mmap.mmap] = {}

    def _map(self, path: Path) -> mmap.mmap:
        if path not in self._maps:
            with open(path, "rb") as handle:
                self._maps[path] = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_READ)
        return self._maps[path]

    def read(self, entry: TensorEntry) -> torch.Tensor:
        count = _numel(entry.shape)
        if count == 0:
            return torch.empty(entry.shape, dtype=entry.dtype)
        view = memoryview(self._map(entry.path))[entry.payload_start + entry.begin : entry.payload_start + entry.end]
        flat = torch.frombuffer(bytearray(view), dtype=entry.dtype, count=count)
        return flat.reshape(entry.shape)

    def close(self) -> None:
        for mapped in self._maps.values():
            mapped.close()
        self._maps.clear()


def read_all(model_dir: Path) -> dict[str, torch.Tensor]:
    """Every tensor of a model folder as host tensors in their stored dtype."""
    entries = read_model_index(model_dir)
    files = TensorFiles()
    try:
        return {name: files.read(entry) for name, entry in entries.items()}
    finally:
        files.close()


def write_file(path: Path, tensors: dict[str, torch.Tensor]) -> None:
    """Write ``tensors`` (host, contiguous) to one safetensors file in name order."""
    header: dict[str, dict] = {}
    offset = 0
    names = sorted(tensors)
    for name in names:
        tensor = tensors[name]
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {tensor.dtype} cannot be stored")
        size = tensor.numel() * tensor.dtype.itemsize
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape), "data_offsets": [offset, offset + size]}
        offset += size
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(text)))
        handle.write(text)
        for name in names:
            tensor = tensors[name].detach().cpu().contiguous()
            handle.write(tensor.reshape(-1).view(torch.uint8).numpy().tobytes() if tensor.numel() else b"")
