"""A decoder made of parts: embedding, blocks run in a listed order, last norm, output head.

The model is data: ``blocks`` (each a ``PreNormBlock`` of parts chosen by the configuration,
layer by layer), ``order`` (which block runs when, and which cache entry it uses) and
``bindings`` (which tensor of the model folder feeds which parameter).  The order may name a
block twice, and a call may read a cache entry that an earlier call fills (``store=False``).
Counterpart of ``Qwen25_15B.forward`` (pico_vllm/model.py:414-445), which loops over a fixed
``ModuleList`` and computes logits for every position; here logits are computed for the
wanted rows only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..errors import ConfigError
from ..parts.base import CacheView, Part


@dataclass(frozen=True)
class LayerCall:
    block: int                 # index into DecoderModel.blocks
    cache: Optional[int]       # index of the cache entry this call uses (None: the mixer keeps nothing)
    store: bool = True         # False: read an entry that an earlier call of the order fills


@dataclass
class Binding:
    part: Part
    names: Dict[str, str]      # the part's piece key -> tensor name in the model folder


class DecoderModel:
    def __init__(self, config, embed: Part, blocks: Sequence, order: Sequence[LayerCall], final_norm: Part,
                 head: Part, bindings: List[Binding], embed_position: Optional[Part] = None):
        """``embed_position``: a position encoding that acts on the residual stream right after the
        embedding (absolute or learned positions): a part with ``add_to(x, positions) -> x`` for the
        float32 stream x [T, width] and int32 positions [T] (-1: a padding row).  Rotary encodings are
        not given here: they belong to the mixer that rotates with them."""
        self.config = config
        self.embed_position = embed_position
        self.embed, self.blocks, self.order = embed, list(blocks), list(order)
        self.final_norm, self.head, self.bindings = final_norm, head, bindings
        self.vocab_size = head.vocab
        self.cache_entries = self._cache_entries()
        self.dtype = None
        self.device = None

    def _cache_entries(self) -> List:
        entries: Dict[int, object] = {}
        filled = set()
        for call in self.order:
            if not 0 <= call.block < len(self.blocks):
                raise ConfigError(f"layer order names block {call.block}, but there are {len(self.blocks)}")
            spec = self.blocks[call.block].mixer.cache_spec()
            if spec is None:
                if call.cache is not None:
                    raise ConfigError(f"block {call.block} keeps no cache but the order gives it entry {call.cache}")
                continue
            if call.cache is None:
                raise ConfigError(f"block {call.block} needs a cache entry")
            if call.cache in entries and entries[call.cache] != spec:
                raise ConfigError(f"cache entry {call.cache} is shared by mixers with different needs")
            entries[call.cache] = spec
            if call.store:
                if call.cache in filled:
                    raise ConfigError(f"cache entry {call.cache} is filled by two calls of the order")
                filled.add(call.cache)
            elif call.cache not in filled:
                raise ConfigError(f"cache entry {call.cache} is read before any call fills it")
        if sorted(entries) != list(range(len(entries))):
            raise ConfigError("cache entries must be numbered 0..n-1 without gaps")
        return [entries[i] for i in range(len(entries))]

    def all_parts(self) -> List[Part]:
        parts = [self.embed] + ([self.embed_position] if self.embed_position is not None else [])
        for b in self.blocks:
            parts.extend(b.parts().values())
        parts += [self.final_norm, self.head]
        return parts

    def materialize(self, device, dtype: torch.dtype) -> None:
        self.device, self.dtype = torch.device(device), dtype
        for p in self.all_parts():
            p.materialize(self.device, dtype)

    def forward(self, batch, views: Sequence[CacheView]) -> torch.Tensor:
        """Runs the batch's tokens through every call of the order; returns float32 logits
        [len(batch.logit_rows), vocab] - or None when ``batch.greedy_out`` was given and the head wrote the
        greedy token of every wanted row there instead."""
        x = self.embed.forward(batch.token_ids, batch.feedback)
        if self.embed_position is not None:
            x = self.embed_position.add_to(x, batch.positions)
        pending = None
        for call in self.order:
            view = None
            if call.cache is not None:
                view = views[call.cache]
                if view.store != call.store:
                    view = CacheView(**{**view.__dict__, "store": call.store})
            x, pending = self.blocks[call.block].forward(x, pending, batch, view)
        if batch.num_logit_rows == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=x.device)
        greedy = getattr(batch, "greedy_out", None) if hasattr(self.head, "greedy") else None
        if pending is None and hasattr(self.head, "can_fuse_norm") \
                and self.head.can_fuse_norm(x, self.final_norm, batch.num_logit_rows):
            if greedy is not None and self.head.greedy(x, self.final_norm, batch.logit_rows, batch.num_logit_rows, greedy):
                return None
            return self.head.forward_normed(x, self.final_norm, batch.logit_rows)
        y = self.final_norm.add_norm(x, pending, rows=batch.logit_rows)
        if greedy is not None and self.head.greedy(y, None, None, batch.num_logit_rows, greedy):
            return None
        return self.head.forward(y)
