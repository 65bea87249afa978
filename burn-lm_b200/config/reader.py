"""Typed reading of config.json keys: every error names the key and says what was wrong."""
from __future__ import annotations

import json
import os
from typing import Any

_MISSING = object()


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


def read_config_json(folder_or_file: str) -> dict:
    path = folder_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path) as f:
            data = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return data


class KeyReader:
    """Reads keys of one JSON object with type checks; `where` prefixes the key in messages."""

    def __init__(self, data: dict, where: str = ""):
        self.data = data
        self.where = where
        self.seen: set[str] = set()

    def _name(self, key):
        return f"{self.where}{key}"

    def _get(self, key, default):
        self.seen.add(key)
        v = self.data.get(key, _MISSING)
        if v is _MISSING or v is None:
            if default is _MISSING:
                raise ConfigError(f"config key '{self._name(key)}' is required")
            return _MISSING
        return v

    def integer(self, key, default: Any = _MISSING, minimum: int | None = None) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                v = int(v)
            else:
                raise ConfigError(f"config key '{self._name(key)}' must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"config key '{self._name(key)}' must be at least {minimum}, got {v}")
        return v

    def number(self, key, default: Any = _MISSING, positive: bool = False) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config key '{self._name(key)}' must be a number, got {v!r}")
        v = float(v)
        if positive and not v > 0:
            raise ConfigError(f"config key '{self._name(key)}' must be positive, got {v}")
        return v

    def boolean(self, key, default: Any = _MISSING) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, bool):
            raise ConfigError(f"config key '{self._name(key)}' must be true or false, got {v!r}")
        return v

    def string(self, key, default: Any = _MISSING) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, str):
            raise ConfigError(f"config key '{self._name(key)}' must be a string, got {v!r}")
        return v

    def obj(self, key, default: Any = _MISSING) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, dict):
            raise ConfigError(f"config key '{self._name(key)}' must be an object, got {v!r}")
        return v

    def int_or_list(self, key, default: Any = _MISSING) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        items = v if isinstance(v, list) else [v]
        for i in items:
            if isinstance(i, bool) or not isinstance(i, int):
                raise ConfigError(f"config key '{self._name(key)}' must be an integer or a list of them, got {v!r}")
        return tuple(items)
