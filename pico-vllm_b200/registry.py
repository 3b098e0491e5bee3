"""One registry from an architecture's name (config.json ``architectures[0]``) to its
configuration class and model builder.  The reference imports its one model class directly
(pico_vllm/run_single.py:2); here every entry point goes through this table."""
from __future__ import annotations

from typing import Callable, Dict, Tuple

from .errors import ConfigError

_ARCHITECTURES: Dict[str, Tuple[type, Callable]] = {}


def register_architecture(name: str, config_cls: type, builder: Callable) -> None:
    """``config_cls.from_dict(raw, where)`` reads config.json; ``builder(config)`` returns a model
    (a ``DecoderModel`` or anything with its interface)."""
    _ARCHITECTURES[name] = (config_cls, builder)


def architectures():
    return sorted(_ARCHITECTURES)


def resolve(name: str) -> Tuple[type, Callable]:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not supported (have {', '.join(architectures())})")
    return _ARCHITECTURES[name]


def config_from_dict(raw: dict, where: str = "config.json"):
    """Typed configuration for whatever architecture ``raw`` names."""
    from .config.base import architecture_name
    cfg_cls, _ = resolve(architecture_name(raw, where))
    return cfg_cls.from_dict(raw, where)


def build_model(config):
    _, builder = resolve(config.architecture)
    return builder(config)


def _register_builtin() -> None:
    from .config.qwen2 import Qwen2Config
    from .models.qwen2 import build_qwen2
    register_architecture("Qwen2ForCausalLM", Qwen2Config, build_qwen2)


_register_builtin()
