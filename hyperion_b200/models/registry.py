"""The one registry from an architecture's name to its configuration type and its model.

``config.json`` names the architecture in ``architectures``; the entry registered under that name
turns the parsed file into a typed configuration and the configuration into a
:class:`~hyperion_b200.parts.spec.ModelSpec`.  The reference keeps the same kind of table from a
model id to its compiler class, filled as a side effect of importing the architecture modules, and
raises for an unknown id (ignition/src/hyperion_ignition/compiler/registry.py:15-31).
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from ..config.base import ConfigError, read_json
from ..parts.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    read_config: Callable[[dict], Any]  # parsed config.json -> typed configuration
    build_spec: Callable[[Any], ModelSpec]  # typed configuration -> model as data
    write_config: Callable[[Any], dict]  # typed configuration -> config.json document


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(architecture: Architecture) -> None:
    if architecture.name in _ARCHITECTURES and _ARCHITECTURES[architecture.name] is not architecture:
        raise ValueError(f"architecture {architecture.name!r} is already registered")
    _ARCHITECTURES[architecture.name] = architecture


def architecture_of(document: dict) -> Architecture:
    names = document.get("architectures")
    if not isinstance(names, list) or not names:
        raise ConfigError("architectures", f"must be a non-empty list, got {names!r}")
    for name in names:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    raise ConfigError("architectures", f"{names!r} is not supported; known: {sorted(_ARCHITECTURES)}")


def get_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise KeyError(f"architecture {name!r} is not registered; known: {sorted(_ARCHITECTURES)}")
    return _ARCHITECTURES[name]


def read_model_config(model_dir: Path) -> tuple[Architecture, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in model folder {model_dir}")
    document = read_json(path)
    architecture = architecture_of(document)
    return architecture, architecture.read_config(document)
