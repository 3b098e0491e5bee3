"""Gated feed-forward: down( act(gate(h)) * up(h) ) with gate and up as one matrix.

pico_vllm/model.py:309-318 (fused gate_up projection, silu(gate) * up, down projection);
the activation runs in float32 as in pico_vllm/kernels/swiglu.py:28-44.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from ..errors import ConfigError
from .base import Param, Part, Piece
from .registry import register


@register("feed_forward", "gated_mlp")
class GatedMLP(Part):
    fuses_residual = True   # forward(..., residual=x) may add its output to x and return None

    def __init__(self, width: int, inner: int, act: str = "silu"):
        if act != "silu":
            raise ConfigError(f"gated_mlp: activation {act!r} is not built (only 'silu')")
        self.width, self.inner = width, inner
        self.gate_up_weight = self.down_weight = None

    def params(self) -> List[Param]:
        return [Param("gate_up_weight", (Piece("gate.weight", (self.inner, self.width)),
                                         Piece("up.weight", (self.inner, self.width)))),
                Param("down_weight", (Piece("down.weight", (self.width, self.inner)),))]

    def can_fuse_norm(self, x: torch.Tensor, norm) -> bool:
        return getattr(norm, "plain_rms", False) and getattr(norm, "weight", None) is not None and self.inner % 8 == 0 \
            and ops.skinny_norm_takes(x, self.gate_up_weight)

    def forward(self, h: Optional[torch.Tensor], batch, residual: Optional[torch.Tensor] = None, norm=None):
        """Returns what is to be added to the residual stream - or, when ``residual`` is given
        and the fused small-batch kernels take the sizes, adds it there itself and returns None.
        With ``norm`` (after ``can_fuse_norm``), ``h`` is None and the normed input is computed from
        ``residual`` inside the first kernel."""
        if norm is not None:
            a = ops.skinny_gate_up_swiglu(residual, self.gate_up_weight, norm.weight, norm.eps)
        elif ops.skinny_takes(h, self.gate_up_weight) and self.inner % 8 == 0:
            a = ops.skinny_gate_up_swiglu(h, self.gate_up_weight)      # product and activation in one kernel
        elif h.shape[0] >= ops.TC_PAIR_MIN_TOKENS and ops.tc_takes(h, self.gate_up_weight) and self.inner % 8 == 0:
            # many tokens: tcgen05 product with the activation in its epilogue (the [T, 2I] buffer never exists);
            # below that the library product and the activation kernel are faster (measured, see ops)
            a = ops.tc_gate_up_swiglu(h, self.gate_up_weight)
        else:
            gu = ops.linear(h, self.gate_up_weight)
            a = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
            ops.swiglu(gu, a)
        if residual is not None and ops.skinny_takes(a, self.down_weight):
            ops.skinny_linear_residual(a, self.down_weight, residual)
            return None
        return ops.linear(a, self.down_weight)
