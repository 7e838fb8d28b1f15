"""Typed reading of a Hugging Face style ``config.json``.

Every value a model needs is read from the file through :class:`ConfigReader`, which names the
offending key in its error instead of substituting a default.  The reference reads its model
configuration the same way: positive integers and finite positive numbers are checked one by one
and a missing required key is an error (ignition/src/hyperion_ignition/compiler/model_config.py:70-80,
:96-169).
"""
from __future__ import annotations

import json
import math
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type, or asks for something unsupported."""

    def __init__(self, key: str, message: str):
        super().__init__(f"config.json: {key!r} {message}")
        self.key = key


class ConfigReader:
    """Wraps the parsed JSON document and hands out checked values."""

    def __init__(self, document: dict[str, Any]):
        if not isinstance(document, dict):
            raise ConfigError("<root>", "must be a JSON object")
        self.document = document

    def has(self, key: str) -> bool:
        return key in self.document and self.document[key] is not None

    def raw(self, key: str, default: Any = None) -> Any:
        return self.document.get(key, default)

    def positive_int(self, key: str) -> int:
        value = self.document.get(key)
        if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
            raise ConfigError(key, f"must be a positive integer, got {value!r}")
        return value

    def positive_number(self, key: str, value: Any = None) -> float:
        if value is None:
            value = self.document.get(key)
        if isinstance(value, bool) or not isinstance(value, (int, float)) or not value > 0 or math.isinf(value):
            raise ConfigError(key, f"must be a finite positive number, got {value!r}")
        return float(value)

    def boolean(self, key: str) -> bool:
        value = self.document.get(key)
        if not isinstance(value, bool):
            raise ConfigError(key, f"must be stated as true or false, got {value!r}")
        return value

    def token_ids(self, key: str) -> tuple[int, ...]:
        value = self.document.get(key)
        if value is None:
            return ()
        items = value if isinstance(value, list) else [value]
        if any(isinstance(i, bool) or not isinstance(i, int) or i < 0 for i in items):
            raise ConfigError(key, f"must be a non-negative integer or a list of them, got {value!r}")
        return tuple(items)


def read_json(path: Path) -> dict[str, Any]:
    with open(path, "r", encoding="utf-8") as handle:
        return json.load(handle)
