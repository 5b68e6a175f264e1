"""Typed reading of a checkpoint's config.json.

A model configuration is a frozen dataclass whose fields are the architecture's
own config.json keys.  `ConfigReader` collects every problem of a dictionary
(missing keys, wrong types, values out of range) and raises them together as one
`ConfigError`, so that a bad config.json is fixed in one pass.
"""
from __future__ import annotations

import json
import os
from typing import Any


class ConfigError(ValueError):
    """config.json lacks a key, or holds a value the engine cannot run."""


_MISSING = object()


class ConfigReader:
    def __init__(self, raw: dict, where: str = "config.json"):
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: expected a JSON object, got {type(raw).__name__}")
        self.raw = raw
        self.where = where
        self.problems: list[str] = []

    def _get(self, key: str, default: Any, kind, check=None):
        value = self.raw.get(key, _MISSING)
        if value is _MISSING or value is None:
            if default is _MISSING:
                self.problems.append(f"missing key '{key}'")
                return None
            return default
        if kind is float and isinstance(value, int) and not isinstance(value, bool):
            value = float(value)
        if kind is int and isinstance(value, bool) or not isinstance(value, kind):
            self.problems.append(f"'{key}' must be {kind.__name__}, got {value!r}")
            return default if default is not _MISSING else None
        if check is not None:
            complaint = check(value)
            if complaint:
                self.problems.append(f"'{key}' = {value!r}: {complaint}")
        return value

    def integer(self, key: str, default: Any = _MISSING, minimum: int = 1):
        return self._get(key, default, int, lambda v: None if v >= minimum else f"must be >= {minimum}")

    def number(self, key: str, default: Any = _MISSING, positive: bool = True):
        return self._get(key, default, float, lambda v: None if (v > 0 or not positive) else "must be > 0")

    def boolean(self, key: str, default: Any = _MISSING):
        return self._get(key, default, bool)

    def optional_integer(self, key: str):
        return self._get(key, None, int)

    def complain(self, text: str) -> None:
        self.problems.append(text)

    def finish(self) -> None:
        if self.problems:
            raise ConfigError(f"{self.where}: " + "; ".join(self.problems))


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file (a model folder holds config.json and model.safetensors)")
    with open(path, "r", encoding="utf-8") as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
