"""Configuration, registry, weight loading and its errors (CPU)."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import helpers
from pico_vllm_b200.config import EngineConfig, Qwen2Config, read_config_json
from pico_vllm_b200.errors import ConfigError, WeightError
from pico_vllm_b200.models import DecoderModel, LayerCall
from pico_vllm_b200.registry import architectures, build_model, config_from_dict, resolve
from pico_vllm_b200.weights import check_tensors, load_weights, wanted_tensors, write_random_model

RAW = helpers.TINY["a"]["raw"]


def test_config_reads_every_size_from_its_keys():
    cfg = config_from_dict(dict(RAW, head_dim=32, eos_token_id=[7, 9], bos_token_id=1))
    assert isinstance(cfg, Qwen2Config)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers) == (256, 64, 2)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (4, 2, 32)
    assert cfg.queries_per_kv == 2 and cfg.eos_token_id == 7 and cfg.bos_token_id == 1
    assert cfg.layer_windows == (None, None)
    assert config_from_dict(dict(RAW)).head_dim == 16          # hidden // heads when not given


def test_config_windows():
    b = helpers.tiny_config("b")
    assert b.layer_windows == (None, 24, 24)
    c = config_from_dict(dict(helpers.TINY["b"]["raw"], layer_types=["sliding_attention", "full_attention",
                                                                      "sliding_attention"]))
    assert c.layer_windows == (24, None, 24)
    assert config_from_dict(c.to_dict()) == c                   # round trip through config.json


@pytest.mark.parametrize("change,word", [
    (dict(hidden_size="64"), "hidden_size"), (dict(vocab_size=None), "vocab_size"),
    (dict(num_key_value_heads=3), "num_key_value_heads"), (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rope_scaling={"type": "yarn", "factor": 4}), "rope_scaling"), (dict(rms_norm_eps=0), "rms_norm_eps"),
    (dict(use_sliding_window=True, sliding_window=None), "sliding_window"),
    (dict(architectures=["LlamaForCausalLM"]), "LlamaForCausalLM"), (dict(architectures=[]), "architectures"),
    (dict(tie_word_embeddings="yes"), "tie_word_embeddings"), (dict(hidden_size=66), "head_dim"),
])
def test_config_errors_name_the_key(change, word):
    raw = dict(RAW, **change)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert word in str(e.value)


def test_registry():
    assert "Qwen2ForCausalLM" in architectures()
    cfg_cls, builder = resolve("Qwen2ForCausalLM")
    model = builder(cfg_cls.from_dict(RAW))
    assert isinstance(model, DecoderModel) and len(model.blocks) == 2
    assert [c.block for c in model.order] == [0, 1] and len(model.cache_entries) == 2
    with pytest.raises(ConfigError):
        resolve("NoSuchModel")


def test_engine_config_checks():
    assert EngineConfig(dtype="bf16").dtype == "bfloat16" and EngineConfig(dtype="fp32").dtype == "float32"
    with pytest.raises(ConfigError):
        EngineConfig(dtype="float16")
    with pytest.raises(ConfigError):
        EngineConfig(page_size=0)


def test_layer_order_is_data():
    cfg = helpers.tiny_config("a")
    m = build_model(cfg)
    # a block twice with a cache entry of its own, and a call that reads another call's entry
    m2 = DecoderModel(cfg, m.embed, m.blocks, [LayerCall(0, 0), LayerCall(1, 1), LayerCall(1, 2), LayerCall(0, 0, store=False)],
                      m.final_norm, m.head, m.bindings)
    assert len(m2.cache_entries) == 3
    with pytest.raises(ConfigError):
        DecoderModel(cfg, m.embed, m.blocks, [LayerCall(0, 0, store=False)], m.final_norm, m.head, m.bindings)
    with pytest.raises(ConfigError):
        DecoderModel(cfg, m.embed, m.blocks, [LayerCall(0, 0), LayerCall(1, 0)], m.final_norm, m.head, m.bindings)
    with pytest.raises(ConfigError):
        DecoderModel(cfg, m.embed, m.blocks, [LayerCall(5, 0)], m.final_norm, m.head, m.bindings)


def test_random_model_folder_round_trip(tmp_path):
    for name, dtype in (("a", "bfloat16"), ("b", "float32")):
        d = helpers.write_tiny_model(name, tmp_path / name, dtype=dtype)
        cfg = config_from_dict(read_config_json(d))
        import dataclasses
        assert dataclasses.replace(cfg, torch_dtype="bfloat16") == helpers.tiny_config(name)
        assert cfg.torch_dtype == dtype
        files = load_file(os.path.join(d, "model.safetensors"))
        model = build_model(cfg)
        assert set(files) == set(wanted_tensors(model))
        assert all(t.dtype == getattr(torch, dtype) for t in files.values())
        # the same seed gives the same tensors; another seed does not
        again = load_file(os.path.join(write_random_model(cfg, helpers.TINY[name]["seed"], str(tmp_path / "again")),
                                       "model.safetensors"))
        if dtype == "bfloat16":
            assert all(torch.equal(files[k], again[k]) for k in files)
        load_weights(model, d, torch.bfloat16, "cpu")
        attn = model.blocks[0].mixer
        nq = cfg.num_attention_heads * cfg.head_dim
        assert attn.qkv_weight.shape == ((cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim,
                                         cfg.hidden_size)
        assert torch.equal(attn.qkv_weight[:nq].float(), files["model.layers.0.self_attn.q_proj.weight"].float())
        assert torch.equal(model.blocks[0].feed_forward.gate_up_weight[cfg.intermediate_size:].float(),
                           files["model.layers.0.mlp.up_proj.weight"].float())
        # storage rule: 16-bit stays bfloat16, 32-bit stays float32, vectors are float32
        assert attn.qkv_weight.dtype == getattr(torch, dtype)
        assert attn.qkv_bias.dtype == torch.float32 and model.blocks[0].norm1.weight.dtype == torch.float32
        norm_w = files["model.layers.0.input_layernorm.weight"].float()
        assert abs(float(norm_w.mean()) - 1.0) < 0.05            # norm weights are 1 + N(0, 0.02)
        load_weights(model, d, torch.float32, "cpu")
        assert attn.qkv_weight.dtype == torch.float32


def test_weight_errors_list_everything_at_once(tmp_path):
    d = helpers.write_tiny_model("b", tmp_path / "m", dtype="float32")
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["lm_head.weight"]
    t["model.layers.0.self_attn.k_proj.bias"] = torch.zeros(5)
    t["model.layers.2.self_attn.o_proj.weight"] = torch.zeros(192, 191)
    t["model.layers.9.extra.weight"] = torch.zeros(3)
    save_file(t, path)
    model = build_model(config_from_dict(read_config_json(d)))
    with pytest.raises(WeightError) as e:
        load_weights(model, d, torch.float32, "cpu")
    err = e.value
    assert err.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == ["model.layers.0.self_attn.k_proj.bias", "model.layers.2.self_attn.o_proj.weight"]
    text = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (2)", "expected [96]", "[192, 191]"):
        assert word in text


def test_tied_model_may_carry_a_head_and_untied_must(tmp_path):
    d = helpers.write_tiny_model("a", tmp_path / "m", dtype="float32")
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    save_file(t, path)
    model = build_model(config_from_dict(read_config_json(d)))
    load_weights(model, d, torch.float32, "cpu")                 # tied: the extra head is ignored
    assert model.head.tied_to is model.embed


def test_folder_errors(tmp_path):
    with pytest.raises(ConfigError):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(RAW))
    model = build_model(config_from_dict(read_config_json(str(tmp_path))))
    with pytest.raises(WeightError):
        load_weights(model, str(tmp_path), torch.float32, "cpu")          # no safetensors file
    (tmp_path / "model.safetensors").write_bytes(b"\x00" * 10)
    with pytest.raises(WeightError):
        load_weights(model, str(tmp_path), torch.float32, "cpu")          # truncated file


def test_no_cpu_path_in_the_product():
    from pico_vllm_b200 import ops
    from pico_vllm_b200.errors import KernelError
    with pytest.raises(KernelError):
        ops.swiglu(torch.zeros(2, 8), torch.zeros(2, 4))


def test_cli_random_model(tmp_path):
    from pico_vllm_b200.cli import main
    cfg_path = tmp_path / "c.json"
    cfg_path.write_text(json.dumps(helpers.TINY["c"]["raw"]))
    assert main(["random-model", "--config", str(cfg_path), "--seed", "4", "--out", str(tmp_path / "m")]) == 0
    cfg = config_from_dict(read_config_json(str(tmp_path / "m")))
    assert cfg.head_dim == 48 and cfg.vocab_size == 331
