"""Configuration of the Qwen2 dense decoder, read from its config.json keys.

Key names and meanings follow the reference's dataclass (pico_vllm/model.py:15-26:
vocab_size, hidden_size, num_hidden_layers, num_attention_heads,
num_key_value_heads, intermediate_size, rms_norm_eps, rope_theta,
max_position_embeddings, tie_word_embeddings) and its derived sizes
(head_dim = hidden_size // num_attention_heads, pico_vllm/model.py:36-38;
query heads per key/value head, pico_vllm/model.py:41-43).  The reference fixes
the other choices in code: a bias on q/k/v only (pico_vllm/model.py:147-152), SiLU
(pico_vllm/model.py:318), half-split rotation over the whole head
(pico_vllm/model.py:116-123).  The window keys (use_sliding_window,
sliding_window, max_window_layers, layer_types) are keys of this architecture's
config.json that the reference never reads; here they choose, layer by layer,
between attention over all keys and over the last ``sliding_window`` keys.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Dict, Optional, Tuple

from ..errors import ConfigError
from .base import KeyReader

ARCHITECTURE = "Qwen2ForCausalLM"


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    hidden_act: str
    # one entry per layer: None = every earlier key is visible, W = the last W keys
    layer_windows: Tuple[Optional[int], ...]
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    architecture = ARCHITECTURE

    @property
    def queries_per_kv(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str = "config.json") -> "Qwen2Config":
        r = KeyReader(raw, where)
        vocab = r.integer("vocab_size", minimum=1)
        hidden = r.integer("hidden_size", minimum=1)
        layers = r.integer("num_hidden_layers", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", default=heads, minimum=1)
        inter = r.integer("intermediate_size", minimum=1)
        eps = r.number("rms_norm_eps", default=1e-6, positive=True)
        theta = r.number("rope_theta", default=1000000.0, positive=True)
        max_pos = r.integer("max_position_embeddings", default=32768, minimum=1)
        tie = r.boolean("tie_word_embeddings", default=True)
        act = r.string("hidden_act", default="silu")
        head_dim = r.integer("head_dim", default=None, minimum=1)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(
                    f"{where}: 'hidden_size' ({hidden}) is not a multiple of 'num_attention_heads' "
                    f"({heads}) and no 'head_dim' is given"
                )
            head_dim = hidden // heads
        if heads % kv_heads != 0:
            raise ConfigError(
                f"{where}: 'num_attention_heads' ({heads}) must be a multiple of "
                f"'num_key_value_heads' ({kv_heads})"
            )
        if head_dim % 2 != 0:
            raise ConfigError(f"{where}: 'head_dim' ({head_dim}) must be even for rotary pairs")
        if act != "silu":
            raise ConfigError(f"{where}: 'hidden_act' must be 'silu' for {ARCHITECTURE}, got {act!r}")
        scaling = r.any("rope_scaling")
        if scaling is not None:
            kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
            if kind != "default":
                raise ConfigError(f"{where}: 'rope_scaling' {scaling!r} is not supported (only null)")
        if r.any("use_mrope", False):
            raise ConfigError(f"{where}: 'use_mrope' = true is not supported")

        use_window = r.boolean("use_sliding_window", default=False)
        window = r.integer("sliding_window", default=None, minimum=1)
        max_window_layers = r.integer("max_window_layers", default=layers, minimum=0)
        layer_types = r.any("layer_types")
        if layer_types is not None:
            if not isinstance(layer_types, list) or len(layer_types) != layers:
                raise ConfigError(f"{where}: 'layer_types' must list one type per layer ({layers})")
            windows = []
            for i, t in enumerate(layer_types):
                if t == "full_attention":
                    windows.append(None)
                elif t == "sliding_attention":
                    if window is None:
                        raise ConfigError(
                            f"{where}: layer {i} is 'sliding_attention' but 'sliding_window' is missing"
                        )
                    windows.append(window)
                else:
                    raise ConfigError(f"{where}: 'layer_types'[{i}] = {t!r} is not a known layer type")
        elif use_window:
            if window is None:
                raise ConfigError(f"{where}: 'use_sliding_window' is true but 'sliding_window' is missing")
            # layers from index max_window_layers on look at a window, the ones below at everything
            windows = [window if i >= max_window_layers else None for i in range(layers)]
        else:
            windows = [None] * layers
        dtype = r.string("torch_dtype", default=None) or r.string("dtype", default="bfloat16")
        return cls(
            vocab_size=vocab,
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=inter,
            rms_norm_eps=eps,
            rope_theta=theta,
            max_position_embeddings=max_pos,
            tie_word_embeddings=tie,
            hidden_act=act,
            layer_windows=tuple(windows),
            bos_token_id=_token_id(r, "bos_token_id"),
            eos_token_id=_token_id(r, "eos_token_id"),
            torch_dtype=dtype,
        )

    def to_dict(self) -> Dict[str, Any]:
        """config.json content that :meth:`from_dict` reads back to an equal object."""
        d = asdict(self)
        windows = d.pop("layer_windows")
        d["architectures"] = [ARCHITECTURE]
        d["model_type"] = "qwen2"
        sizes = {w for w in windows if w is not None}
        if len(sizes) > 1:
            raise ConfigError("config.json of this architecture holds one 'sliding_window' size only")
        if sizes:
            d["use_sliding_window"] = True
            d["sliding_window"] = sizes.pop()
            d["layer_types"] = [
                "full_attention" if w is None else "sliding_attention" for w in windows
            ]
        else:
            d["use_sliding_window"] = False
        return {k: v for k, v in d.items() if v is not None}


def _token_id(r: KeyReader, key: str) -> Optional[int]:
    v = r.any(key)
    if isinstance(v, list):  # some folders list several end tokens; the first one is used
        v = v[0] if v else None
    if v is None:
        return None
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"{r.where}: key '{key}' must be an integer, got {v!r}")
    return v
