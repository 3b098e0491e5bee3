"""Registries of part kinds by name, so that a configuration can choose them layer by layer
and a user can add kinds of their own without touching this package."""
from __future__ import annotations

from typing import Callable, Dict

from ..errors import ConfigError

MIXERS: Dict[str, Callable] = {}
FEED_FORWARDS: Dict[str, Callable] = {}
NORMS: Dict[str, Callable] = {}
POSITIONS: Dict[str, Callable] = {}

_TABLES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position": POSITIONS}


def register(kind: str, name: str):
    """Decorator: ``@register("mixer", "my_mixer")`` above a class makes ``make("mixer",
    "my_mixer", **sizes)`` build it."""
    if kind not in _TABLES:
        raise ConfigError(f"unknown kind of part {kind!r} (have {sorted(_TABLES)})")

    def deco(cls):
        _TABLES[kind][name] = cls
        return cls
    return deco


def make(kind: str, name: str, **kwargs):
    table = _TABLES[kind]
    if name not in table:
        raise ConfigError(f"no {kind} named {name!r} is registered (have {sorted(table)})")
    return table[name](**kwargs)
