from .decoder import DecoderModel, LayerCall, Binding
from .qwen2 import build_qwen2

__all__ = ["DecoderModel", "LayerCall", "Binding", "build_qwen2"]
