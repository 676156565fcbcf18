"""Typed access to the keys of a config.json.

The reference reads config.json through a reader whose errors name the key and the kind of value found, and
which treats a JSON null as an absent key
(evidence/pipeline/onboarding/Starlings.Roost.Onboarding/HfConfig.cs:35-192). This is the same idea for the
serving path: no caller indexes the raw dict.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot be served; the message names the key."""


def _kind(v: Any) -> str:
    if isinstance(v, bool):
        return "a boolean"
    if isinstance(v, int):
        return "an integer"
    if isinstance(v, float):
        return "a number"
    if isinstance(v, str):
        return "a string"
    if isinstance(v, list):
        return "a list"
    if isinstance(v, dict):
        return "an object"
    return "null"


class ConfigReader:
    def __init__(self, values: dict, source: str = "config.json"):
        if not isinstance(values, dict):
            raise ConfigError(f"{source}: the top level is {_kind(values)}; expected an object")
        self._v = values
        self.source = source
        self.read: set[str] = set()

    @classmethod
    def from_path(cls, path) -> "ConfigReader":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        try:
            values = json.loads(path.read_text())
        except FileNotFoundError:
            raise ConfigError(f"{path}: no such file") from None
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
        return cls(values, str(path))

    def has(self, key: str) -> bool:
        return self._v.get(key) is not None

    def raw(self, key: str):
        self.read.add(key)
        return self._v.get(key)

    def _fail(self, key: str, v: Any, want: str):
        raise ConfigError(f"{self.source}: key '{key}' is {_kind(v)} ({v!r}); expected {want}")

    def opt_int(self, key: str) -> int | None:
        v = self.raw(key)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            self._fail(key, v, "an integer")
        return int(v)

    def required_int(self, key: str) -> int:
        v = self.opt_int(key)
        if v is None:
            raise ConfigError(f"{self.source}: required key '{key}' is absent")
        return v

    def positive_int(self, key: str, default: int | None = None) -> int:
        v = self.opt_int(key)
        if v is None:
            if default is None:
                raise ConfigError(f"{self.source}: required key '{key}' is absent")
            v = default
        if v <= 0:
            raise ConfigError(f"{self.source}: key '{key}' is {v}; it must be positive")
        return v

    def opt_float(self, key: str) -> float | None:
        v = self.raw(key)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            self._fail(key, v, "a number")
        return float(v)

    def opt_bool(self, key: str) -> bool | None:
        v = self.raw(key)
        if v is None:
            return None
        if not isinstance(v, bool):
            self._fail(key, v, "a boolean")
        return v

    def opt_str(self, key: str) -> str | None:
        v = self.raw(key)
        if v is None:
            return None
        if not isinstance(v, str):
            self._fail(key, v, "a string")
        return v

    def opt_strs(self, key: str) -> list[str] | None:
        v = self.raw(key)
        if v is None:
            return None
        if not isinstance(v, list) or not all(isinstance(s, str) for s in v):
            self._fail(key, v, "a list of strings")
        return list(v)

    def opt_ints(self, key: str) -> list[int] | None:
        v = self.raw(key)
        if v is None:
            return None
        if isinstance(v, int) and not isinstance(v, bool):
            return [v]
        if not isinstance(v, list) or not all(isinstance(s, int) and not isinstance(s, bool) for s in v):
            self._fail(key, v, "an integer or a list of integers")
        return list(v)

    def opt_object(self, key: str) -> "ConfigReader | None":
        v = self.raw(key)
        if v is None:
            return None
        if not isinstance(v, dict):
            self._fail(key, v, "an object")
        return ConfigReader(v, f"{self.source}: {key}")
