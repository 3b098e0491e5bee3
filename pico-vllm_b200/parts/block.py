"""Arrangement of parts in one layer: pre-norm residual block.

x += mixer(norm1(x)); x += feed_forward(norm2(x))  (pico_vllm/model.py:361-374).  The adds are
not done here: a block hands the not-yet-added output of its feed-forward to whoever norms next
(the next block or the last norm), so that every add is fused into a norm kernel.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .base import CacheView, Part


class PreNormBlock:
    def __init__(self, norm1: Part, mixer: Part, norm2: Part, feed_forward: Part):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self):
        return {"norm1": self.norm1, "mixer": self.mixer, "norm2": self.norm2, "feed_forward": self.feed_forward}

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], batch,
                cache: CacheView) -> Tuple[torch.Tensor, torch.Tensor]:
        """x: float32 residual stream [T, width]; pending: output of the previous part that is
        still to be added to x (or None).  Returns (x, pending) in the same sense."""
        h = self.norm1.add_norm(x, pending)
        a = self._call(self.mixer, x, h, batch, cache)
        h = self.norm2.add_norm(x, a)
        return x, self._call(self.feed_forward, x, h, batch)

    @staticmethod
    def _call(part, x, *args):
        # a part that says ``fuses_residual`` may add its output to x itself and return None
        if getattr(part, "fuses_residual", False):
            return part.forward(*args, residual=x)
        return part.forward(*args)
