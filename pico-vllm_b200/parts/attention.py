"""Grouped-query attention over the paged cache: the mixer of this architecture.

qkv projection (bias added inside the rotary kernel) -> rotation of q and k and store of k, v
into pages (one kernel) -> paged causal attention (optionally over a window) -> output
projection.  Same order as pico_vllm/model.py:200-227 (projection, split, RoPE, cache store,
paged attention, o_proj); scale head_dim^-1/2 (pico_vllm/kernels/attention.py:92,231).  One
code path serves portions of prompts and single decoded tokens; the reference has three
(pico_vllm/model.py:186-302).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import ops
from .base import CacheView, MixerPlan, PagedKV, Param, Part, Piece, StepShape
from .registry import register


@dataclass(frozen=True)
class AttentionPlan(MixerPlan):
    splits: int = 1            # parts each single token's key range is cut into
    pair_min_keys: int = 0     # > 0: prompt attention gives every query tile two blocks, which share a tile
                               # that sees at least this many keys (two partial results per token and head in scratch)


@register("mixer", "gqa_attention")
class GQAAttention(Part):
    fuses_residual = True   # forward(..., residual=x) may add its output to x and return None

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, position: Part,
                 qkv_bias: bool = True, window: Optional[int] = None, scale: Optional[float] = None):
        self.width, self.n_heads, self.n_kv_heads, self.head_dim = width, n_heads, n_kv_heads, head_dim
        self.position, self.has_bias, self.window = position, qkv_bias, window
        self.scale = head_dim ** -0.5 if scale is None else scale
        self.qkv_weight = self.qkv_bias = self.o_weight = None

    def params(self) -> List[Param]:
        q, kv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        ps = [Param("qkv_weight", (Piece("q.weight", (q, self.width)), Piece("k.weight", (kv, self.width)),
                                   Piece("v.weight", (kv, self.width)))),
              Param("o_weight", (Piece("o.weight", (self.width, q)),))]
        if self.has_bias:
            ps.append(Param("qkv_bias", (Piece("q.bias", (q,)), Piece("k.bias", (kv,)), Piece("v.bias", (kv,))),
                            kind="vector"))
        return ps

    def cache_spec(self):
        return PagedKV(self.n_kv_heads, self.head_dim, self.window)

    def materialize(self, device, dtype):
        self.position.materialize(device, dtype)

    # ------------------------------------------------------------------ launch policy of the attention kernels
    def plan_key(self):
        return ("gqa_attention", self.n_heads, self.n_kv_heads, self.head_dim, self.window)

    def plan(self, shape: StepShape) -> AttentionPlan:
        splits = self._splits(shape)
        pair = self._pair_min_keys(shape)
        parts = max(splits, 2) if pair > 0 else splits
        scratch = ops.attention_scratch_floats(shape.num_tokens, self.n_heads, self.head_dim, parts)
        return AttentionPlan(key=(splits, pair), scratch_floats=scratch, splits=splits, pair_min_keys=pair)

    def _splits(self, shape: StepShape) -> int:
        """How many parts to cut each single token's key range into: a power of two (the parts of one
        token and kv head run as one thread-block cluster): up to 16 while that is at most one block
        per SM, else up to 8 while the blocks make no more than one wave of two per SM; each part at
        least two tiles of 64 keys."""
        groups = max(1, shape.num_tokens * self.n_kv_heads)
        want = 16 if groups * 16 <= shape.num_sms else min(2 * shape.num_sms // groups, 8)
        want = min(want, shape.max_kv // 128)
        splits = 1
        while splits * 2 <= want:
            splits *= 2
        return splits

    def _pair_min_keys(self, shape: StepShape) -> int:
        """Whether prompt attention should give every query tile two blocks (the threshold in keys, or 0):
        only when every portion of the step comes after a long context (``pair_min_context`` of the engine
        configuration), where a tile takes long enough to pay for the pair, and when the tiles are too few
        to keep the SMs busy by themselves (under two per SM)."""
        m = getattr(shape.engine, "pair_min_context", 0)
        portions = [(n, st) for n, st in zip(shape.q_lens, shape.starts) if n > 1]
        if not (m > 0 and portions and shape.num_sms > 1 and getattr(shape.engine, "dtype", "") == "bfloat16"
                and min(st for _, st in portions) >= m):
            return 0
        tiles = len(portions) * self.n_heads * -(-max(n for n, _ in portions) // 128)
        return m if tiles <= 2 * shape.num_sms else 0

    def can_fuse_norm(self, x: torch.Tensor, norm) -> bool:
        """True when forward can take the residual stream itself and apply ``norm`` inside its
        first kernel (small batches)."""
        return getattr(norm, "plain_rms", False) and getattr(norm, "weight", None) is not None \
            and ops.skinny_norm_takes(x, self.qkv_weight)

    def forward(self, h: Optional[torch.Tensor], batch, cache: CacheView, residual: Optional[torch.Tensor] = None,
                norm=None):
        """Returns what is to be added to the residual stream - or, when ``residual`` is given
        and the fused small-batch kernels take the sizes, adds it there itself and returns None.
        With ``norm`` (after ``can_fuse_norm``), ``h`` is None and the normed input is computed from
        ``residual`` inside the first kernel."""
        gb = batch.groups[cache.group]
        slots = gb.slots if cache.store else None
        plan = batch.plan(self)
        pairing = getattr(self.position, "pairing", "half")
        splits, pair_min_keys = (plan.splits, plan.pair_min_keys) if plan is not None else (1, 0)
        if norm is not None:
            qkv = ops.skinny_qkv_rope_store(residual, self.qkv_weight, self.qkv_bias, batch.positions,
                                            self.position.inv_freq, slots, cache.k, cache.v, self.n_heads,
                                            self.n_kv_heads, self.head_dim, cache.page_size, norm.weight, norm.eps,
                                            pairing=pairing)
            h = qkv             # only its dtype and device are used below
        elif ops.skinny_takes(h, self.qkv_weight):
            # a handful of tokens: projection, bias, rotation and cache store are one kernel
            qkv = ops.skinny_qkv_rope_store(h, self.qkv_weight, self.qkv_bias, batch.positions,
                                            self.position.inv_freq, slots, cache.k, cache.v, self.n_heads,
                                            self.n_kv_heads, self.head_dim, cache.page_size, pairing=pairing)
        else:
            qkv = ops.linear(h, self.qkv_weight)
            ops.rope_store(qkv, self.qkv_bias, batch.positions, self.position.inv_freq, slots, cache.k, cache.v,
                           self.n_heads, self.n_kv_heads, self.head_dim, cache.page_size, pairing=pairing)
        out = torch.empty((h.shape[0], self.n_heads * self.head_dim), dtype=h.dtype, device=h.device)
        if ops.mma_attention_takes(h.dtype, self.n_heads, self.n_kv_heads, self.head_dim):
            ops.paged_attention_mma(qkv, cache.k, cache.v, out, batch.tok_seg, batch.positions, gb.block_table,
                                    batch.cu_q, batch.prefill_segs, batch.num_prefill_segs, batch.max_prefill_q,
                                    batch.decode_tokens, batch.num_decode_tokens, self.n_heads, self.n_kv_heads,
                                    self.head_dim, cache.page_size, self.window, self.scale, splits,
                                    batch.scratch, cache.k_map, cache.v_map, cache.k_map2d, cache.v_map2d,
                                    pair_min_keys)
        else:       # float32, or sizes the tensor-core kernels do not take
            ops.paged_attention(qkv, cache.k, cache.v, out, batch.tok_seg, batch.positions, gb.block_table,
                                self.n_heads, self.n_kv_heads, self.head_dim, cache.page_size, self.window,
                                self.scale, splits, batch.scratch)
        if residual is not None and ops.skinny_takes(out, self.o_weight):
            ops.skinny_linear_residual(out, self.o_weight, residual)
            return None
        return ops.linear(out, self.o_weight)
