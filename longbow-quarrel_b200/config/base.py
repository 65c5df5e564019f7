"""What every architecture's configuration shares: reading config.json and the
errors that name the offending key."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot be turned into a typed configuration."""


_MISSING = object()


def read_config_json(folder_or_file) -> dict:
    path = Path(folder_or_file)
    if path.is_dir():
        path = path / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json at {path}")
    try:
        data = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON: {exc}") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return data


class KeyReader:
    """Typed access to the keys of a config.json dict."""

    def __init__(self, data: dict, where: str = "config.json"):
        self.data = data
        self.where = where

    def _get(self, key: str, default: Any):
        value = self.data.get(key, _MISSING)
        if value is _MISSING or value is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing")
            return _MISSING
        return value

    def integer(self, key: str, default: Any = _MISSING, minimum: int | None = None):
        value = self._get(key, default)
        if value is _MISSING:
            return default
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value == int(value):
                value = int(value)
            else:
                raise ConfigError(f"{self.where}: '{key}' must be an integer, found {value!r}")
        if minimum is not None and value < minimum:
            raise ConfigError(f"{self.where}: '{key}' must be >= {minimum}, found {value}")
        return value

    def number(self, key: str, default: Any = _MISSING, positive: bool = False):
        value = self._get(key, default)
        if value is _MISSING:
            return default
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"{self.where}: '{key}' must be a number, found {value!r}")
        value = float(value)
        if positive and not value > 0:
            raise ConfigError(f"{self.where}: '{key}' must be > 0, found {value}")
        return value

    def boolean(self, key: str, default: Any = _MISSING):
        value = self._get(key, default)
        if value is _MISSING:
            return default
        if not isinstance(value, bool):
            raise ConfigError(f"{self.where}: '{key}' must be true or false, found {value!r}")
        return value

    def string(self, key: str, default: Any = _MISSING):
        value = self._get(key, default)
        if value is _MISSING:
            return default
        if not isinstance(value, str):
            raise ConfigError(f"{self.where}: '{key}' must be a string, found {value!r}")
        return value

    def int_or_list(self, key: str) -> tuple[int, ...]:
        value = self.data.get(key)
        if value is None:
            return ()
        if isinstance(value, int) and not isinstance(value, bool):
            return (value,)
        if isinstance(value, list) and all(isinstance(v, int) and not isinstance(v, bool) for v in value):
            return tuple(value)
        raise ConfigError(f"{self.where}: '{key}' must be an integer or a list of integers, found {value!r}")
