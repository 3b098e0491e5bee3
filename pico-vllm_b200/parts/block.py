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
        a = self._run(self.norm1, self.mixer, x, pending, batch, cache)
        return x, self._run(self.norm2, self.feed_forward, x, a, batch)

    @staticmethod
    def _run(norm, part, x, pending, *args):
        """norm, then the part.  A part that says ``fuses_residual`` may add its output to x itself
        and return None; one that also has ``can_fuse_norm`` may take x and the norm instead of
        normed activations (when nothing is pending to be added first)."""
        fuses = getattr(part, "fuses_residual", False)
        if fuses and pending is None and hasattr(part, "can_fuse_norm") and part.can_fuse_norm(x, norm):
            return part.forward(None, *args, residual=x, norm=norm)
        h = norm.add_norm(x, pending)
        if fuses:
            return part.forward(h, *args, residual=x)
        return part.forward(h, *args)
