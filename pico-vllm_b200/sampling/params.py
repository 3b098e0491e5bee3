"""Sampling options, with the reference's names and meanings: ``max_new_tokens``,
``temperature`` (0 = greedy argmax) and ``top_p`` (>= 1 = off) are the arguments of its
``Engine.submit`` (pico_vllm/engine.py:243-247) and of ``sampler.sample``
(pico_vllm/sampler.py:91-107).  ``seed`` and ``ignore_eos`` are additions: the reference draws
from torch's global generator and always stops at the tokenizer's end token."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..errors import ConfigError


@dataclass
class SamplingParams:
    max_new_tokens: int = 16
    temperature: float = 1.0
    top_p: float = 1.0
    seed: Optional[int] = None
    ignore_eos: bool = False
    max_tokens: Optional[int] = None     # another name for max_new_tokens

    def __post_init__(self):
        if self.max_tokens is not None:
            self.max_new_tokens = self.max_tokens
        if self.max_new_tokens < 1:
            raise ConfigError("max_new_tokens must be at least 1")
        if self.temperature < 0:
            raise ConfigError("temperature must be >= 0 (0 means greedy)")
        if not self.top_p > 0:
            raise ConfigError("top_p must be > 0")
