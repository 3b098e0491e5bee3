"""Puts the pieces together: model folder -> model with weights -> cache -> step function.

The reference does this inline in its entry script (pico_vllm/run_single.py:10-29: config,
model, load_weights, .to(bf16).to("cuda"), BlockManager with 500 pages of 16 tokens, Engine).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..cache.manager import CacheManager
from ..config.base import read_config_json
from ..config.engine import EngineConfig
from ..errors import ConfigError, KernelError, OutOfPages
from ..registry import build_model, config_from_dict
from ..weights.loader import load_weights, load_state_dict
from .runner import ModelRunner

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _prepare_precision(dtype: str) -> None:
    # float32 matrix products must be true float32: no TF32, no reduced-precision reductions
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")


def _require_device(device) -> None:
    """Says in the engine's own words that there is no GPU, before torch says it in its own."""
    if torch.device(device).type == "cuda" and not torch.cuda.is_available():
        raise KernelError("no CUDA device: this engine runs on a GPU only (there is no CPU path)")


def load_model(model_dir: str, cfg: EngineConfig):
    """Model of the folder's architecture with its weights on the device."""
    _require_device(cfg.device)
    config = config_from_dict(read_config_json(model_dir), where=f"{model_dir}/config.json")
    model = build_model(config)
    _prepare_precision(cfg.dtype)
    dtype = TORCH_DTYPES[cfg.dtype]
    load_weights(model, model_dir, dtype, cfg.device)
    model.materialize(cfg.device, dtype)
    return model


def model_from_tensors(config, tensors, cfg: EngineConfig):
    """Same from a configuration object and tensors in memory (name -> tensor)."""
    _require_device(cfg.device)
    model = build_model(config)
    _prepare_precision(cfg.dtype)
    dtype = TORCH_DTYPES[cfg.dtype]
    load_state_dict(model, tensors, dtype, cfg.device)
    model.materialize(cfg.device, dtype)
    return model


def max_model_len(model, cfg: EngineConfig) -> int:
    limit = getattr(model.config, "max_position_embeddings", None)
    if cfg.max_model_len is not None:
        if limit is not None and cfg.max_model_len > limit:
            raise ConfigError(f"max_model_len {cfg.max_model_len} exceeds the model's "
                              f"max_position_embeddings {limit}")
        return cfg.max_model_len
    return limit if limit is not None else 4096


def make_cache(model, cfg: EngineConfig, poison_freed: bool = False) -> CacheManager:
    """Cache manager sized by ``num_pages``, else by ``max_cache_tokens``, else by free memory."""
    dtype = TORCH_DTYPES[cfg.dtype]
    longest = max_model_len(model, cfg)
    if cfg.num_pages is not None:
        pages = cfg.num_pages
    elif cfg.max_cache_tokens is not None:
        pages = -(-cfg.max_cache_tokens // cfg.page_size)
    else:
        probe = CacheManager(model.cache_entries, cfg.page_size, 1, 1, cfg.page_size, dtype, "cpu", allocate=False)
        per_page = max(1, probe.bytes_per_page())
        dev = torch.device(cfg.device)
        if dev.type == "cuda":
            free, _ = torch.cuda.mem_get_info(dev)
            budget = int(free * 0.5)
        else:
            budget = 256 << 20
        pages = max(1, budget // per_page)
        # no more than every request at full length needs
        pages = min(pages, cfg.max_num_seqs * -(-longest // cfg.page_size))
    if cfg.max_cache_tokens is not None or cfg.num_pages is not None:
        longest = min(longest, pages * cfg.page_size)
    if pages < 1:
        raise OutOfPages("the cache would have no page")
    return CacheManager(model.cache_entries, cfg.page_size, pages, cfg.max_num_seqs, longest, dtype,
                        cfg.device, poison_freed=poison_freed)


def make_runner(model_dir: str, cfg: EngineConfig, poison_freed: bool = False) -> ModelRunner:
    model = load_model(model_dir, cfg)
    return ModelRunner(model, make_cache(model, cfg, poison_freed), cfg)
