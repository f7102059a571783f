"""Typed reading of an architecture's config.json.

The reference reads eight keys by substring search with an integer/decimal
scanner that has no exponent support (src/model.cpp:328-353, 366-379) and keeps
every other size as a compile-time constant (src/config.h:29-50).  Here every
size comes from config.json through a real JSON parse, each key is read with a
stated type, and an error names the key.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type, or asks for something unsupported."""


_MISSING = object()


class KeyReader:
    """Reads keys of one JSON object with type checks; remembers which keys were used."""

    def __init__(self, data: dict[str, Any], where: str = "config.json"):
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: expected a JSON object")
        self.data = data
        self.where = where

    def _get(self, key: str, default: Any):
        if key in self.data and self.data[key] is not None:
            return self.data[key]
        if default is _MISSING:
            raise ConfigError(f"{self.where}: required key '{key}' is missing")
        return default

    def integer(self, key: str, default: Any = _MISSING, *, minimum: int | None = None):
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: key '{key}' must be an integer, found {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: key '{key}' must be >= {minimum}, found {v}")
        return v

    def number(self, key: str, default: Any = _MISSING, *, positive: bool = False):
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: key '{key}' must be a number, found {v!r}")
        v = float(v)
        if positive and not v > 0:
            raise ConfigError(f"{self.where}: key '{key}' must be > 0, found {v}")
        return v

    def boolean(self, key: str, default: Any = _MISSING):
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, found {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING):
        v = self._get(key, default)
        if v is not None and not isinstance(v, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, found {v!r}")
        return v

    def string_list(self, key: str, default: Any = _MISSING):
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, list) or not all(isinstance(s, str) for s in v):
            raise ConfigError(f"{self.where}: key '{key}' must be a list of strings, found {v!r}")
        return tuple(v)

    def int_or_int_list(self, key: str, default: Any = _MISSING):
        v = self._get(key, default)
        if v is None:
            return ()
        if isinstance(v, int) and not isinstance(v, bool):
            return (v,)
        if isinstance(v, list) and all(isinstance(i, int) and not isinstance(i, bool) for i in v):
            return tuple(v)
        raise ConfigError(f"{self.where}: key '{key}' must be an integer or a list of integers, found {v!r}")


class ModelConfig:
    """Base of every architecture's typed configuration.

    Subclasses are frozen dataclasses with ``from_dict`` (config.json keys in)
    and ``to_dict`` (the same keys out, so a model folder can be written from a
    configuration)."""

    architecture: str

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict[str, Any]:
        raise NotImplementedError


def load_config_dict(model_dir) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        data = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return data
