"""Reading and writing the safetensors container without any helper library.

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

MAX_HEADER_BYTES = 64 << 20

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


class _DuplicateKey(Exception):
    pass


def _object_without_duplicates(pairs: list[tuple[str, object]]) -> dict:
    """A JSON object as a dict; a name that comes twice is an error, not the last value winning
    (the reference refuses duplicate tensor names: helios/crates/helios-hal/src/weights_plan.rs:52-90)."""
    found: dict = {}
    for key, value in pairs:
        if key in found:
            raise _DuplicateKey(key)
        found[key] = value
    return found


def read_header(path: Path) -> dict[str, TensorEntry]:
    """The tensors one file declares, checked against the file's size."""
    path = Path(path)
    size = path.stat().st_size
    with open(path, "rb") as handle:
        prefix = handle.read(8)
        if len(prefix) != 8:
            raise SafetensorsError(f"{path.name}: shorter than its 8-byte header length")
        (header_len,) = struct.unpack("<Q", prefix)
        if header_len > MAX_HEADER_BYTES or 8 + header_len > size:
            raise SafetensorsError(f"{path.name}: header length {header_len} does not fit the file ({size} bytes)")
        try:
            document = json.loads(handle.read(header_len).decode("utf-8"), object_pairs_hook=_object_without_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise SafetensorsError(f"{path.name}: header is not JSON ({error})") from None
        except _DuplicateKey as error:
            raise SafetensorsError(f"{path.name}: the header names {error.args[0]!r} twice") from None
    if not isinstance(document, dict):
        raise SafetensorsError(f"{path.name}: header must be a JSON object")
    payload = size - 8 - header_len
    entries: dict[str, TensorEntry] = {}
    for name, meta in document.items():
        if name == "__metadata__":
            continue
        try:
            dtype_name, shape, (begin, end) = meta["dtype"], tuple(meta["shape"]), meta["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path.name}: tensor {name!r} lacks dtype, shape or data_offsets") from None
        if dtype_name not in _DTYPES:
            raise SafetensorsError(f"{path.name}: tensor {name!r} has unsupported dtype {dtype_name!r}")
        dtype = _DTYPES[dtype_name]
        if any(isinstance(e, bool) or not isinstance(e, int) or e < 0 for e in shape):
            raise SafetensorsError(f"{path.name}: tensor {name!r} has a bad shape {shape!r}")
        if not (0 <= begin <= end <= payload):
            raise SafetensorsError(f"{path.name}: tensor {name!r} range [{begin}, {end}) lies outside the payload ({payload} bytes)")
        if end - begin != _numel(shape) * dtype.itemsize:
            raise SafetensorsError(
                f"{path.name}: tensor {name!r} holds {end - begin} bytes but shape {list(shape)} of {dtype_name} needs {_numel(shape) * dtype.itemsize}"
            )
        entries[name] = TensorEntry(name, dtype, shape, begin, end, path, 8 + header_len)
    ordered = sorted(entries.values(), key=lambda e: (e.begin, e.end))
    for before, after in zip(ordered, ordered[1:]):
        if after.begin < before.end:
            raise SafetensorsError(f"{path.name}: tensors {before.name!r} and {after.name!r} overlap")
    return entries


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
