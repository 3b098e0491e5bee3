"""Weights from safetensors files by tensor name.

The model says which tensors it wants (its ``bindings``: part, piece key -> tensor name) and
what shape each must have.  The loader looks at the names and shapes in the folder first and
raises ONE :class:`WeightError` that lists every missing tensor, every unexpected tensor and
every wrong shape; only then does it read, fuse and place tensors.  Pieces of one parameter are
concatenated along dimension 0 (q, k, v -> qkv; gate, up -> gate_up), as the reference does
(pico_vllm/weights.py:42-43,58); the reference checks nothing (a missing name is a bare
KeyError, shapes are never compared, pico_vllm/weights.py:18-68).

Storage rule: matrices stay bfloat16 when stored in 16 bits and stay float32 when stored in 32
bits; vectors (norm weights, biases) are float32; integer tables would be int32.  With
``dtype=float32`` everything floating is float32.
"""
from __future__ import annotations

import glob
import json
import os
from typing import Dict, List, Tuple

import torch

from ..errors import WeightError


class TensorFiles:
    """All ``*.safetensors`` files of a folder, opened lazily, addressed by tensor name."""

    def __init__(self, model_dir: str):
        from safetensors import safe_open
        files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
        if not files:
            raise WeightError(f"{model_dir}: no .safetensors file in this folder")
        self._handles = []
        self.where: Dict[str, int] = {}
        for path in files:
            try:
                h = safe_open(path, framework="pt", device="cpu")
            except Exception as e:  # a truncated or foreign file
                raise WeightError(f"{path}: cannot be read as safetensors ({e})") from None
            self._handles.append(h)
            for name in h.keys():
                self.where[name] = len(self._handles) - 1

    def names(self) -> List[str]:
        return sorted(self.where)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self._handles[self.where[name]].get_slice(name).get_shape())

    def tensor(self, name: str) -> torch.Tensor:
        return self._handles[self.where[name]].get_tensor(name)


def wanted_tensors(model) -> Dict[str, Tuple[int, ...]]:
    """Tensor name -> shape the model needs, from its bindings."""
    want: Dict[str, Tuple[int, ...]] = {}
    for b in model.bindings:
        for param in b.part.params():
            for piece in param.pieces:
                if piece.key not in b.names:
                    raise WeightError(f"model builder gave no tensor name for '{piece.key}' of {type(b.part).__name__}")
                want[b.names[piece.key]] = tuple(piece.shape)
    return want


def check_tensors(model, have: Dict[str, Tuple[int, ...]], where: str) -> None:
    """Raises one WeightError naming all missing, unexpected and wrongly shaped tensors."""
    want = wanted_tensors(model)
    ignorable = getattr(model, "ignorable_tensors", set())
    missing = sorted(n for n in want if n not in have)
    unexpected = sorted(n for n in have if n not in want and n not in ignorable)
    wrong = sorted((n, have[n], want[n]) for n in want if n in have and tuple(have[n]) != want[n])
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: the tensors do not match the model"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " +
                     ", ".join(f"{n} is {list(h)}, expected {list(w)}" for n, h, w in wrong))
    err = WeightError("\n".join(lines))
    err.missing, err.unexpected, err.wrong_shape = missing, unexpected, [w[0] for w in wrong]
    raise err


def _place(t: torch.Tensor, kind: str, mode: torch.dtype, name: str) -> torch.Tensor:
    if not t.is_floating_point():
        return t.to(torch.int32)
    if kind == "vector" or mode == torch.float32:
        return t.to(torch.float32)
    if t.dtype == torch.float32 or t.dtype == torch.float64:
        return t.to(torch.float32)          # stored in 32-bit: stays so
    return t.to(torch.bfloat16)


def load_weights(model, model_dir: str, dtype: torch.dtype, device) -> None:
    """Reads the folder's tensors into the model's parts on ``device``."""
    files = TensorFiles(model_dir)
    have = {n: files.shape(n) for n in files.names()}
    check_tensors(model, have, model_dir)
    load_from(model, files.tensor, dtype, device)


def load_from(model, get_tensor, dtype: torch.dtype, device) -> None:
    """Fills the model's parameters from ``get_tensor(name) -> torch.Tensor`` (already checked)."""
    for b in model.bindings:
        for param in b.part.params():
            pieces = [_place(get_tensor(b.names[p.key]), param.kind, dtype, b.names[p.key]) for p in param.pieces]
            if len({p.dtype for p in pieces}) > 1:
                pieces = [p.to(torch.float32) for p in pieces]
            t = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=0)
            b.part.assign(param.attr, t.contiguous().to(device))


def load_state_dict(model, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
    """Same as :func:`load_weights` from tensors in memory (name -> tensor)."""
    check_tensors(model, {n: tuple(t.shape) for n, t in tensors.items()}, "state dict")
    load_from(model, tensors.__getitem__, dtype, device)
