from .base import KeyReader, read_config_json, architecture_name
from .qwen2 import Qwen2Config
from .engine import EngineConfig, canonical_dtype

__all__ = ["KeyReader", "read_config_json", "architecture_name", "Qwen2Config", "EngineConfig",
           "canonical_dtype"]
