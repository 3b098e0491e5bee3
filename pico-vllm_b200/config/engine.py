"""Settings of the engine itself (cache, scheduler, precision), apart from the model's.

The reference spreads these over constructor arguments and inline constants
(pico_vllm/engine.py:15-31, pico_vllm/run_single.py:17-29: 500 pages of 16
tokens, at most 4 running requests, graph batch 8, max_seq_len 4096).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

from ..errors import ConfigError

DTYPES = ("bfloat16", "float32")


def canonical_dtype(name: str) -> str:
    table = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp32": "float32", "float32": "float32",
             "float": "float32"}
    if name not in table:
        raise ConfigError(f"dtype must be one of bfloat16, float32 (got {name!r})")
    return table[name]


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"            # "bfloat16": serving kernels; "float32": everything in true 32-bit
    page_size: int = 16                # tokens per cache page (pico_vllm/model.py:33)
    num_pages: Optional[int] = None    # pages per layer group; None = sized from max_cache_tokens
    max_cache_tokens: Optional[int] = None  # tokens the pool must hold when num_pages is None
    max_num_seqs: int = 4              # running requests at a time (pico_vllm/scheduler.py:84)
    max_num_batched_tokens: int = 2048  # token budget of one step
    prefill_chunk: Optional[int] = None  # longest portion of one prompt in a step (None = the budget)
    max_model_len: Optional[int] = None  # longest request; None = max_position_embeddings
    use_cuda_graph: bool = True        # replay decode-only steps from a CUDA graph (pico_vllm/engine.py:98-137)
    graph_batch_sizes: Tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64)
    # a step that is one full portion of one prompt is replayed from a graph too (long prompts come as a row of
    # such steps): its number of tokens; None = the longest portion (prefill_chunk or the budget), 0 = never
    graph_prefill_tokens: Optional[int] = None
    # portions of prompts whose requests already hold at least this many tokens get two blocks per query tile in
    # attention, half of the keys each (a few long tiles would otherwise set the kernel's time); 0 = never
    pair_min_context: int = 6144
    async_scheduling: bool = True      # launch a step before the tokens of the step before are read
    seed: int = 0
    device: str = "cuda:0"

    def __post_init__(self):
        self.dtype = canonical_dtype(self.dtype)
        if self.page_size < 1:
            raise ConfigError("page_size must be >= 1")
        if self.max_num_seqs < 1:
            raise ConfigError("max_num_seqs must be >= 1")
        if self.max_num_batched_tokens < 1:
            raise ConfigError("max_num_batched_tokens must be >= 1")
        if self.prefill_chunk is not None and self.prefill_chunk < 1:
            raise ConfigError("prefill_chunk must be >= 1")
