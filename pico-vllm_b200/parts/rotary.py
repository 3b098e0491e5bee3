"""Rotary position encoding: the frequencies a mixer's fused kernel rotates with.

inv_freq_i = theta^(-2i/rot_dim), angle = position * inv_freq_i, pairs (d, d + head_dim/2)
(pico_vllm/model.py:80-90, 116-123): ``pairing = "half"``, the only pairing the kernels have; a
position part may name another (``"interleaved"``: pairs (2i, 2i+1)) and the kernels then refuse it
with a KernelError instead of rotating wrongly.  The reference looks angles up in a table of cos/sin that
ends up in bfloat16 (pico_vllm/run_single.py:13); here the kernel computes them in float32
from the position.  ``rot_dim`` below ``head_dim`` rotates only the first rot_dim/2 pairs;
:class:`NoPosition` rotates nothing.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from .base import Part
from .registry import register


@register("position", "rotary")
class Rotary(Part):
    pairing = "half"

    def __init__(self, head_dim: int, theta: float, rot_dim: int = None, pairing: str = "half"):
        self.head_dim, self.theta, self.pairing = head_dim, theta, pairing
        self.rot_dim = head_dim if rot_dim is None else rot_dim
        if self.rot_dim % 2 or self.rot_dim > head_dim:
            raise ConfigError(f"rotary: rot_dim {self.rot_dim} must be even and at most head_dim {head_dim}")
        self.inv_freq = None

    def frequencies(self) -> torch.Tensor:
        # the same float32 expression as the reference (pico_vllm/model.py:80-82)
        return 1.0 / (self.theta ** (torch.arange(0, self.rot_dim, 2).float() / self.rot_dim))

    def materialize(self, device, dtype):
        self.inv_freq = self.frequencies().to(device)


@register("position", "none")
class NoPosition(Part):
    pairing = "half"

    def __init__(self, head_dim: int = 0, **_):
        self.head_dim, self.rot_dim = head_dim, 0
        self.inv_freq = None

    def materialize(self, device, dtype):
        self.inv_freq = torch.zeros(0, dtype=torch.float32, device=device)
