"""pico-vllm_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

From a model folder (config.json + model.safetensors) to generated tokens:
typed configuration and a registry of architectures (``config``, ``registry``),
weights by tensor name (``weights``), layers put together from parts (``parts``,
``models``), a paged cache manager (``cache``), one step function and a
scheduler above it (``engine``), sampling (``sampling``), and hand-written CUDA
kernels (``csrc``, called through ``ops``).
"""
__version__ = "0.1.0"

from .errors import (PicoError, ConfigError, WeightError, OutOfPages, KernelError, ScheduleError)

__all__ = ["PicoError", "ConfigError", "WeightError", "OutOfPages", "KernelError", "ScheduleError",
           "LLM", "SamplingParams", "EngineConfig"]


def __getattr__(name):
    # the entry points import torch and the CUDA extension; load them on first use
    if name in ("LLM", "SamplingParams"):
        from .engine import llm
        return getattr(llm, name)
    if name == "EngineConfig":
        from .config import EngineConfig
        return EngineConfig
    raise AttributeError(name)
