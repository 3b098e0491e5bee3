"""Typed reading of config.json.

Every architecture has one frozen dataclass whose fields are filled from that
architecture's own config.json keys by :class:`KeyReader`.  The reader checks the
type of each value, names the key in every error, and remembers which keys it was
asked for, so that a config class can tell unknown keys from known ones.

The reference has no such layer: its ``ModelConfig`` is a dataclass of defaults
that never reads config.json (pico_vllm/model.py:15-55).
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Optional

from ..errors import ConfigError

_MISSING = object()


class KeyReader:
    """Reads typed values out of a config.json dictionary."""

    def __init__(self, raw: Dict[str, Any], where: str = "config.json"):
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.raw = raw
        self.where = where
        self.seen = set()

    def _get(self, key: str, default: Any):
        self.seen.add(key)
        if key not in self.raw or self.raw[key] is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing")
            return default
        return self.raw[key]

    def integer(self, key: str, default: Any = _MISSING, minimum: Optional[int] = None):
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: key '{key}' must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: key '{key}' must be >= {minimum}, got {v}")
        return v

    def number(self, key: str, default: Any = _MISSING, positive: bool = False):
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: key '{key}' must be a number, got {v!r}")
        v = float(v)
        if positive and not v > 0.0:
            raise ConfigError(f"{self.where}: key '{key}' must be > 0, got {v}")
        return v

    def boolean(self, key: str, default: Any = _MISSING):
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING):
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, got {v!r}")
        return v

    def any(self, key: str, default: Any = None):
        return self._get(key, default)


def read_config_json(model_dir: str) -> Dict[str, Any]:
    """Returns the parsed config.json of a model folder."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json in this folder")
    try:
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None


def architecture_name(raw: Dict[str, Any], where: str = "config.json") -> str:
    """The model class name config.json asks for: ``architectures[0]``."""
    archs = raw.get("architectures")
    if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError(
            f"{where}: key 'architectures' must be a list with exactly one model class name, got {archs!r}"
        )
    return archs[0]
