"""RMS norm on the float32 residual stream, fused with the residual add that precedes it.

y = x * rsqrt(mean(x^2) + eps) * w in float32 (pico_vllm/RMSNorm.py:22-34; plain form
pico_vllm/model.py:57-66).  The reference adds the residual in a separate torch op
(pico_vllm/model.py:372-373); here the add and the norm are one kernel.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Param, Part, Piece
from .registry import register


@register("norm", "rmsnorm")
class RMSNorm(Part):
    # y = x * rsqrt(mean(x^2) + eps) * weight and nothing else: what the product kernels with the norm inside
    # compute.  A part that takes a norm into its own kernel asks for this mark, not for attribute names.
    plain_rms = True

    def __init__(self, width: int, eps: float):
        self.width, self.eps = width, eps
        self.weight: Optional[torch.Tensor] = None
        self.act_dtype = torch.bfloat16

    def params(self) -> List[Param]:
        return [Param("weight", (Piece("weight", (self.width,)),), kind="vector", init="one_plus_normal")]

    def materialize(self, device, dtype):
        self.act_dtype = dtype

    def add_norm(self, x: torch.Tensor, delta: Optional[torch.Tensor],
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: float32 [T, width] residual stream, updated in place by ``x += delta`` unless
        ``rows`` picks rows (then x stays).  Returns norm(x) in the activation dtype."""
        n = rows.shape[0] if rows is not None else x.shape[0]
        out = torch.empty((n, self.width), dtype=self.act_dtype, device=x.device)
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
