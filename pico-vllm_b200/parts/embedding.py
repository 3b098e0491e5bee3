"""Token embedding and output head.

x = E[ids] (pico_vllm/model.py:405,427) into the float32 residual stream; logits = y . W^T with
W the embedding matrix when tied (pico_vllm/model.py:445) or a matrix of its own (the reference
creates lm_head for the untied case but never uses it, pico_vllm/model.py:409-412; its older
model does, pico_vllm/legacy/model.py:223-226).  Logits are float32 and are computed only for
the rows that were asked for.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Param, Part, Piece


class TokenEmbedding(Part):
    def __init__(self, vocab: int, width: int):
        self.vocab, self.width = vocab, width
        self.weight = None

    def params(self) -> List[Param]:
        return [Param("weight", (Piece("weight", (self.vocab, self.width)),))]

    def forward(self, ids: torch.Tensor, feedback: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = torch.empty((ids.shape[0], self.width), dtype=torch.float32, device=ids.device)
        return ops.embedding(ids, self.weight, out, feedback)


class OutputHead(Part):
    def __init__(self, vocab: int, width: int, tied_to: Optional[TokenEmbedding] = None):
        self.vocab, self.width, self.tied_to = vocab, width, tied_to
        self.weight = None

    def params(self) -> List[Param]:
        if self.tied_to is not None:
            return []
        return [Param("weight", (Piece("weight", (self.vocab, self.width)),))]

    def matrix(self) -> torch.Tensor:
        return self.tied_to.weight if self.tied_to is not None else self.weight

    def forward(self, y: torch.Tensor) -> torch.Tensor:
        return ops.logits_linear(y, self.matrix())

    def can_fuse_norm(self, x: torch.Tensor, norm, n_rows: int) -> bool:
        return getattr(norm, "plain_rms", False) and getattr(norm, "weight", None) is not None \
            and ops.skinny_norm_takes(x, self.matrix(), n_rows)

    def forward_normed(self, x: torch.Tensor, norm, rows: torch.Tensor) -> torch.Tensor:
        """Logits of rows ``rows`` of the residual stream x, with the last norm applied inside the kernel."""
        return ops.skinny_linear(x, self.matrix(), None, torch.float32, norm.weight, norm.eps, rows)

    def greedy(self, x: torch.Tensor, norm, rows: Optional[torch.Tensor], n_rows: int, out: torch.Tensor) -> bool:
        """The greedy tokens of ``n_rows`` rows straight into ``out`` (int32), without logits: argmax in the
        product's epilogue.  With ``norm``, x is the residual stream and the last norm runs inside the kernel
        (``rows`` picks its rows); without, x is already normed.  False when the fused kernel does not take
        the sizes: the caller then computes logits."""
        w = self.matrix()
        if norm is not None:
            if not self.can_fuse_norm(x, norm, n_rows):
                return False
            ops.skinny_argmax(x, w, out, norm.weight, norm.eps, rows)
            return True
        if not ops.skinny_takes(x, w):
            return False
        ops.skinny_argmax(x, w, out)
        return True
