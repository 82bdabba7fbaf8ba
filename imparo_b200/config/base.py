"""Reading config.json into typed values.

The reference builds its typed plan from a model file's metadata keys and reports a
missing key by name (imparo-model/src/lib.rs:582-600, PlanError::MissingMetadata /
Inconsistent).  Here the source is the architecture's own config.json.
"""
from __future__ import annotations

import json
import os
from typing import Any, Iterable, Optional


class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type, or contradicts another."""


_MISSING = object()


class KeyReader:
    """Typed access to a config.json dictionary; every failure names the key."""

    def __init__(self, values: dict, where: str = "config.json"):
        if not isinstance(values, dict):
            raise ConfigError(f"{where}: top level must be an object")
        self.values = values
        self.where = where

    def _get(self, names: Iterable[str], default: Any = _MISSING) -> Any:
        names = tuple(names)
        for n in names:
            if n in self.values and self.values[n] is not None:
                return self.values[n]
        if default is _MISSING:
            raise ConfigError(f"{self.where}: missing required key '{names[0]}'"
                              + (f" (also accepted: {', '.join(names[1:])})" if len(names) > 1 else ""))
        return default

    def integer(self, *names: str, default: Any = _MISSING, minimum: Optional[int] = None) -> int:
        v = self._get(names, default)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and float(v).is_integer():
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: key '{names[0]}' must be an integer, found {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: key '{names[0]}' must be >= {minimum}, found {v}")
        return int(v)

    def number(self, *names: str, default: Any = _MISSING) -> float:
        v = self._get(names, default)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: key '{names[0]}' must be a number, found {v!r}")
        return float(v)

    def boolean(self, *names: str, default: Any = _MISSING) -> bool:
        v = self._get(names, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key '{names[0]}' must be true or false, found {v!r}")
        return v

    def strings(self, *names: str, default: Any = _MISSING) -> Optional[tuple]:
        v = self._get(names, default)
        if v is None:
            return None
        if not isinstance(v, (list, tuple)) or not all(isinstance(s, str) for s in v):
            raise ConfigError(f"{self.where}: key '{names[0]}' must be a list of strings")
        return tuple(v)

    def integers(self, *names: str, default: Any = _MISSING) -> Optional[tuple]:
        v = self._get(names, default)
        if v is None:
            return None
        if isinstance(v, int) and not isinstance(v, bool):
            return (int(v),)
        if not isinstance(v, (list, tuple)) or not all(isinstance(s, int) and not isinstance(s, bool) for s in v):
            raise ConfigError(f"{self.where}: key '{names[0]}' must be a list of integers")
        return tuple(int(s) for s in v)

    def raw(self, name: str, default: Any = None) -> Any:
        return self.values.get(name, default)


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json in this model folder")
    with open(path) as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None
