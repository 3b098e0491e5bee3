"""The batch of one step, as the parts see it.

One flat list of tokens made of *segments*: a segment is the next tokens of one request, a
portion of its prompt or one decoded token.  The reference passes the same facts as
``input_ids, position_ids, slot_mapping, block_table, context_lens, new_token_lens,
q_start_loc`` (pico_vllm/model.py:414-425) but never mixes prompts and decoding in one batch
(pico_vllm/engine.py:299-357 vs 402-410).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class GroupBatch:
    slots: torch.Tensor          # int32 [T]: cache row of each token's key/value in this group (-1: none)
    block_table: torch.Tensor    # int32 [S, max_blocks]: page of each block of each segment's request


@dataclass
class Batch:
    num_tokens: int
    num_segments: int
    token_ids: torch.Tensor      # int32 [T]
    positions: torch.Tensor      # int32 [T]: absolute position of each token in its request (-1: padding)
    tok_seg: torch.Tensor        # int32 [T]: segment of each token
    seg_slots: torch.Tensor      # int32 [S]: request slot of each segment (row of fixed-size state)
    cu_q: torch.Tensor           # int32 [S+1]: first token of each segment
    logit_rows: torch.Tensor     # int32 [R]: tokens whose logits are wanted
    num_logit_rows: int
    groups: Dict[int, GroupBatch]
    q_lens: List[int]            # host copy: tokens of each segment
    kv_lens: List[int]           # host copy: length of each segment's request after this step
    # what each mixer planned for this step (Part.plan), by the mixer's plan_key(), and the float32 scratch
    # that the step function provides for all of them (the largest any plan asked for; None if none did)
    plans: Dict[object, object] = field(default_factory=dict)
    scratch: Optional[torch.Tensor] = None
    decode_only: bool = False
    # the batch split for kernels that treat portions and single tokens differently
    prefill_segs: Optional[torch.Tensor] = None   # int32: segments with two or more tokens (None: all)
    num_prefill_segs: int = 0
    max_prefill_q: int = 0
    decode_tokens: Optional[torch.Tensor] = None  # int32: tokens of one-token segments (None: every token)
    num_decode_tokens: int = 0
    # tokens chosen by the sampling kernel in the step before; a token id -(j+1) in token_ids means feedback[j]
    feedback: Optional[torch.Tensor] = None
    # int32, one entry per wanted row: when given, the head may write the greedy token of every wanted row here and
    # return no logits
    greedy_out: Optional[torch.Tensor] = None

    def plan(self, mixer):
        """The plan ``mixer.plan(shape)`` returned for this step, or None."""
        return self.plans.get(mixer.plan_key())
