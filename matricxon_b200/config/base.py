"""Typed reading of a model folder's ``config.json``.

The reference reads hyper-parameters ad hoc from GGUF metadata with untyped
getters (app/gguf/metadata.py:23-43, app/architectures/starcoder2.py:63-79).
Here every key is read once, type-checked, and kept in a frozen dataclass; a
missing or ill-typed key is an error that names the key.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot describe a runnable model."""


_MISSING = object()


class ConfigReader:
    """Pulls typed values out of a config dictionary and remembers which keys were read."""

    def __init__(self, raw: dict[str, Any], where: str = "config.json") -> None:
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: expected a JSON object, got {type(raw).__name__}")
        self.raw = raw
        self.where = where
        self.read_keys: set[str] = set()

    def _get(self, key: str, default: Any) -> Any:
        self.read_keys.add(key)
        if key in self.raw and self.raw[key] is not None:
            return self.raw[key]
        if default is _MISSING:
            raise ConfigError(f"{self.where}: required key {key!r} is missing")
        return default

    def integer(self, key: str, default: Any = _MISSING, minimum: int | None = None) -> int:
        value = self._get(key, default)
        if value is None:
            return value
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value.is_integer():
                value = int(value)
            else:
                raise ConfigError(f"{self.where}: {key!r} must be an integer, got {value!r}")
        if minimum is not None and value < minimum:
            raise ConfigError(f"{self.where}: {key!r} must be >= {minimum}, got {value}")
        return value

    def number(self, key: str, default: Any = _MISSING, positive: bool = False) -> float:
        value = self._get(key, default)
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"{self.where}: {key!r} must be a number, got {value!r}")
        value = float(value)
        if positive and not value > 0.0:
            raise ConfigError(f"{self.where}: {key!r} must be > 0, got {value}")
        return value

    def boolean(self, key: str, default: Any = _MISSING) -> bool:
        value = self._get(key, default)
        if not isinstance(value, bool):
            raise ConfigError(f"{self.where}: {key!r} must be true or false, got {value!r}")
        return value

    def string(self, key: str, default: Any = _MISSING) -> str:
        value = self._get(key, default)
        if value is not None and not isinstance(value, str):
            raise ConfigError(f"{self.where}: {key!r} must be a string, got {value!r}")
        return value

    def optional_integer(self, key: str, minimum: int | None = None) -> int | None:
        """A key that may be absent or null; both read as None."""
        self.read_keys.add(key)
        if self.raw.get(key) is None:
            return None
        return self.integer(key, minimum=minimum)


def read_config_json(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        with open(path, "r", encoding="utf-8") as handle:
            raw = json.load(handle)
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from exc
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return raw
