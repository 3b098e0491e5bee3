"""Grouped-query attention over the paged cache: the mixer of this architecture.

qkv projection (bias added inside the rotary kernel) -> rotation of q and k and store of k, v
into pages (one kernel) -> paged causal attention (optionally over a window) -> output
projection.  Same order as pico_vllm/model.py:200-227 (projection, split, RoPE, cache store,
paged attention, o_proj); scale head_dim^-1/2 (pico_vllm/kernels/attention.py:92,231).  One
code path serves portions of prompts and single decoded tokens; the reference has three
(pico_vllm/model.py:186-302).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import CacheView, PagedKV, Param, Part, Piece
from .registry import register


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

    def can_fuse_norm(self, x: torch.Tensor, norm) -> bool:
        """True when forward can take the residual stream itself and apply ``norm`` inside its
        first kernel (small batches)."""
        return hasattr(norm, "eps") and getattr(norm, "weight", None) is not None \
            and ops.skinny_norm_takes(x, self.qkv_weight)

    def forward(self, h: Optional[torch.Tensor], batch, cache: CacheView, residual: Optional[torch.Tensor] = None,
                norm=None):
        """Returns what is to be added to the residual stream - or, when ``residual`` is given
        and the fused small-batch kernels take the sizes, adds it there itself and returns None.
        With ``norm`` (after ``can_fuse_norm``), ``h`` is None and the normed input is computed from
        ``residual`` inside the first kernel."""
        gb = batch.groups[cache.group]
        slots = gb.slots if cache.store else None
        if norm is not None:
            qkv = ops.skinny_qkv_rope_store(residual, self.qkv_weight, self.qkv_bias, batch.positions,
                                            self.position.inv_freq, slots, cache.k, cache.v, self.n_heads,
                                            self.n_kv_heads, self.head_dim, cache.page_size, norm.weight, norm.eps)
            h = qkv             # only its dtype and device are used below
        elif ops.skinny_takes(h, self.qkv_weight):
            # a handful of tokens: projection, bias, rotation and cache store are one kernel
            qkv = ops.skinny_qkv_rope_store(h, self.qkv_weight, self.qkv_bias, batch.positions,
                                            self.position.inv_freq, slots, cache.k, cache.v, self.n_heads,
                                            self.n_kv_heads, self.head_dim, cache.page_size)
        else:
            qkv = ops.linear(h, self.qkv_weight)
            ops.rope_store(qkv, self.qkv_bias, batch.positions, self.position.inv_freq, slots, cache.k, cache.v,
                           self.n_heads, self.n_kv_heads, self.head_dim, cache.page_size)
        out = torch.empty((h.shape[0], self.n_heads * self.head_dim), dtype=h.dtype, device=h.device)
        if ops.mma_attention_takes(h.dtype, self.n_heads, self.n_kv_heads, self.head_dim):
            ops.paged_attention_mma(qkv, cache.k, cache.v, out, batch.tok_seg, batch.positions, gb.block_table,
                                    batch.cu_q, batch.prefill_segs, batch.num_prefill_segs, batch.max_prefill_q,
                                    batch.decode_tokens, batch.num_decode_tokens, self.n_heads, self.n_kv_heads,
                                    self.head_dim, cache.page_size, self.window, self.scale, batch.attn_splits,
                                    batch.scratch, cache.k_map, cache.v_map, cache.k_map2d, cache.v_map2d,
                                    batch.pair_min_keys)
        else:       # float32, or sizes the tensor-core kernels do not take
            ops.paged_attention(qkv, cache.k, cache.v, out, batch.tok_seg, batch.positions, gb.block_table,
                                self.n_heads, self.n_kv_heads, self.head_dim, cache.page_size, self.window,
                                self.scale, batch.attn_splits, batch.scratch)
        if residual is not None and ops.skinny_takes(out, self.o_weight):
            ops.skinny_linear_residual(out, self.o_weight, residual)
            return None
        return ops.linear(out, self.o_weight)
