"""Typed reading of an architecture's config.json.

A model configuration is a frozen dataclass whose fields are the architecture's own
config.json keys.  `ConfigReader` pulls keys out of the parsed JSON with a type and, where the
format defines one, a default; every error names the key.  No model size lives anywhere
else in the package: parts receive their sizes and constants from the configuration.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """config.json is missing a key, has a value of the wrong type, or asks for an option
    this engine does not run."""


_MISSING = object()


class ConfigReader:
    def __init__(self, raw: dict, where: str = "config.json"):
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.raw = raw
        self.where = where
        self.used: set[str] = set()

    def _get(self, key: str, default: Any):
        self.used.add(key)
        v = self.raw.get(key, _MISSING)
        if v is _MISSING or v is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing")
            return default
        return v

    def int(self, key: str, default: Any = _MISSING, *, min: int | None = None) -> int | None:
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{self.where}: '{key}' must be an integer, got {v!r}")
        if min is not None and v < min:
            raise ConfigError(f"{self.where}: '{key}' must be >= {min}, got {v}")
        return v

    def float(self, key: str, default: Any = _MISSING, *, positive: bool = False) -> float | None:
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: '{key}' must be a number, got {v!r}")
        v = float(v)
        if positive and not v > 0:
            raise ConfigError(f"{self.where}: '{key}' must be > 0, got {v}")
        return v

    def bool(self, key: str, default: Any = _MISSING) -> bool:
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: '{key}' must be true or false, got {v!r}")
        return v

    def str(self, key: str, default: Any = _MISSING) -> str | None:
        v = self._get(key, default)
        if v is not None and not isinstance(v, str):
            raise ConfigError(f"{self.where}: '{key}' must be a string, got {v!r}")
        return v

    def any(self, key: str, default: Any = None):
        return self._get(key, default)


def read_config_json(folder) -> dict:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None


def architecture_name(raw: dict) -> str:
    arch = raw.get("architectures")
    if not (isinstance(arch, list) and arch and isinstance(arch[0], str)):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return arch[0]
