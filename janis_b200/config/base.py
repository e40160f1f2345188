"""Reading a model folder's config.json into typed values.

A configuration class states, key by key, what it reads from config.json, the
type it expects and the default it takes when the key is absent.  Nothing else
in the package carries a model size: every part gets its sizes and constants
from a configuration object.

The reference parses config.json into one flat struct with defaults and guards
that return errors instead of panicking (`qwen/config.go:127-270`,
`qwen/config_guard_test.go:17-60`); the helpers here do the same per key.
"""
from __future__ import annotations

import json
import os
from typing import Any, Mapping


class ConfigError(ValueError):
    """config.json is missing, malformed, or describes a model that cannot be built."""


_MISSING = object()


class ConfigReader:
    """Typed access to a parsed config.json; remembers which keys were read."""

    def __init__(self, raw: Mapping[str, Any], where: str = "config.json"):
        if not isinstance(raw, Mapping):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.raw = dict(raw)
        self.where = where
        self.seen: set[str] = set()

    def _get(self, key: str, default: Any) -> Any:
        self.seen.add(key)
        v = self.raw.get(key, _MISSING)
        if v is _MISSING or v is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key {key!r} is missing")
            return default
        return v

    def integer(self, key: str, default: Any = _MISSING, minimum: int | None = None) -> int:
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"{self.where}: {key!r} must be an integer, found {v!r}")
        v = int(v)
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: {key!r} must be >= {minimum}, found {v}")
        return v

    def number(self, key: str, default: Any = _MISSING, minimum: float | None = None,
               exclusive: bool = False) -> float:
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: {key!r} must be a number, found {v!r}")
        v = float(v)
        if minimum is not None and (v < minimum or (exclusive and v == minimum)):
            op = ">" if exclusive else ">="
            raise ConfigError(f"{self.where}: {key!r} must be {op} {minimum}, found {v}")
        return v

    def boolean(self, key: str, default: Any = _MISSING) -> bool:
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: {key!r} must be true or false, found {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING) -> str:
        v = self._get(key, default)
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: {key!r} must be a string, found {v!r}")
        return v

    def int_or_list(self, key: str) -> tuple[int, ...]:
        """A single id or a list of ids (eos_token_id is either; `qwen/config.go:252-261`)."""
        v = self._get(key, ())
        if isinstance(v, bool):
            raise ConfigError(f"{self.where}: {key!r} must be an integer or a list of integers")
        if isinstance(v, int):
            return (v,)
        if isinstance(v, (list, tuple)) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
            return tuple(int(x) for x in v)
        raise ConfigError(f"{self.where}: {key!r} must be an integer or a list of integers, found {v!r}")

    def string_list(self, key: str, default: Any = _MISSING) -> tuple[str, ...]:
        v = self._get(key, default)
        if v is None:
            return ()
        if isinstance(v, (list, tuple)) and all(isinstance(x, str) for x in v):
            return tuple(v)
        raise ConfigError(f"{self.where}: {key!r} must be a list of strings, found {v!r}")

    def has(self, key: str) -> bool:
        return self.raw.get(key) is not None


def read_config_json(model_dir: str) -> dict:
    """Parse <model_dir>/config.json; errors carry the path (`qwen/config.go:128-135`)."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            text = f.read()
    except OSError as e:
        raise ConfigError(f"read config.json: {path}: {e.strerror or e}") from e
    try:
        raw = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"parse config.json: {path}: {e}") from e
    if not isinstance(raw, dict):
        raise ConfigError(f"parse config.json: {path}: top level must be a JSON object")
    return raw
