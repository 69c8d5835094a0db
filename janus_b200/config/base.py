"""Reading typed values out of a config.json dictionary.

Errors name the key, as the reference's `ConfigError` does
(crates/janus-engine/src/model/config.rs:16-35).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional


class ConfigError(ValueError):
    """A config.json that cannot be used: a missing key, a wrong type, a value
    out of range, or an architecture nobody registered."""


_MISSING = object()


def read_config_json(path: str) -> Dict[str, Any]:
    """`path` is a config.json or a folder that holds one
    (crates/janus-engine/src/model/config.rs:114-132)."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r") as f:
            text = f.read()
    except OSError as e:
        raise ConfigError(f"cannot read config file '{path}': {e}") from e
    try:
        data = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"config file '{path}' is not valid JSON: {e}") from e
    if not isinstance(data, dict):
        raise ConfigError(f"config file '{path}' must hold a JSON object")
    return data


class KeyReader:
    """Typed access to the keys of one config dictionary."""

    def __init__(self, data: Dict[str, Any]):
        self.data = data

    def _get(self, key: str, default: Any):
        v = self.data.get(key, _MISSING)
        if v is _MISSING or v is None:
            if default is _MISSING:
                raise ConfigError(f"missing required key '{key}'")
            return _MISSING
        return v

    def integer(self, key: str, default: Any = _MISSING, minimum: Optional[int] = 1) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                v = int(v)
            else:
                raise ConfigError(f"key '{key}' must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"key '{key}' must be at least {minimum}, got {v}")
        return v

    def number(self, key: str, default: Any = _MISSING, positive: bool = True) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"key '{key}' must be a number, got {v!r}")
        v = float(v)
        if positive and not v > 0.0:
            raise ConfigError(f"key '{key}' must be positive, got {v}")
        return v

    def boolean(self, key: str, default: Any = _MISSING) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, bool):
            raise ConfigError(f"key '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING) -> Any:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, str):
            raise ConfigError(f"key '{key}' must be a string, got {v!r}")
        return v

    def id_list(self, key: str) -> tuple:
        """An integer, a list of integers, or absent -> tuple of ints."""
        v = self.data.get(key)
        if v is None:
            return ()
        if isinstance(v, int) and not isinstance(v, bool):
            return (v,)
        if isinstance(v, list) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
            return tuple(v)
        raise ConfigError(f"key '{key}' must be an integer or a list of integers, got {v!r}")
