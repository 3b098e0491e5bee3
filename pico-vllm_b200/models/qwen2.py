"""Qwen2 dense decoder ("Qwen2ForCausalLM") put together from parts.

Layer i = RMSNorm -> grouped-query attention with q/k/v bias and rotary positions -> RMSNorm ->
SwiGLU feed-forward, pre-norm residual (pico_vllm/model.py:340-374); embedding, last norm and
a tied or separate output head (pico_vllm/model.py:402-412).  Tensor names are those the
reference's loader reads (pico_vllm/weights.py:18-68) plus ``lm_head.weight`` for untied models.
"""
from __future__ import annotations

from ..config.qwen2 import Qwen2Config
from ..parts import GQAAttention, GatedMLP, OutputHead, PreNormBlock, RMSNorm, Rotary, TokenEmbedding
from .decoder import Binding, DecoderModel, LayerCall


def build_qwen2(cfg: Qwen2Config) -> DecoderModel:
    H = cfg.hidden_size
    embed = TokenEmbedding(cfg.vocab_size, H)
    bindings = [Binding(embed, {"weight": "model.embed_tokens.weight"})]
    blocks = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        norm1, norm2 = RMSNorm(H, cfg.rms_norm_eps), RMSNorm(H, cfg.rms_norm_eps)
        attn = GQAAttention(H, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                            position=Rotary(cfg.head_dim, cfg.rope_theta), qkv_bias=True,
                            window=cfg.layer_windows[i])
        mlp = GatedMLP(H, cfg.intermediate_size, cfg.hidden_act)
        blocks.append(PreNormBlock(norm1, attn, norm2, mlp))
        bindings += [
            Binding(norm1, {"weight": p + "input_layernorm.weight"}),
            Binding(attn, {f"{n}.{t}": f"{p}self_attn.{n}_proj.{t}" for n in "qkv" for t in ("weight", "bias")}
                    | {"o.weight": p + "self_attn.o_proj.weight"}),
            Binding(norm2, {"weight": p + "post_attention_layernorm.weight"}),
            Binding(mlp, {f"{n}.weight": f"{p}mlp.{n}_proj.weight" for n in ("gate", "up", "down")}),
        ]
    final_norm = RMSNorm(H, cfg.rms_norm_eps)
    bindings.append(Binding(final_norm, {"weight": "model.norm.weight"}))
    head = OutputHead(cfg.vocab_size, H, tied_to=embed if cfg.tie_word_embeddings else None)
    if not cfg.tie_word_embeddings:
        bindings.append(Binding(head, {"weight": "lm_head.weight"}))
    order = [LayerCall(block=i, cache=i) for i in range(cfg.num_hidden_layers)]
    model = DecoderModel(cfg, embed, blocks, order, final_norm, head, bindings)
    # a tied model folder may still carry a copy of the head; it is not an error
    model.ignorable_tensors = {"lm_head.weight"} if cfg.tie_word_embeddings else set()
    return model
