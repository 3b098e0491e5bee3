"""Runs the reference's own pure-torch model on a tiny random Qwen2 and stores its logits.

The reference's current model (pico_vllm/model.py) needs its Triton kernels and a GPU;
its older pure-torch model, pico_vllm/legacy/model.py, imports and runs on the CPU
together with the contiguous cache of pico_vllm/cache.py:22-57.  Its attention begins
with an assert that compares an instance with a class (pico_vllm/legacy/model.py:89),
which only passes with asserts off, so this script re-runs itself under ``python -O``.

    python tests/golden/make_golden.py /path/to/reference

writes tests/golden/legacy_tiny.safetensors with, for two tiny configurations, the
token ids and the legacy model's whole-prompt logits, and its logits when the same
prompt is fed as portions through its cache.  The weights come from
tests/plain_qwen2.random_weights(cfg, seed), so tests can rebuild them.
tests/test_plain.py compares tests/plain_qwen2.py with these numbers.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # name: (config kwargs, seed, prompt length, portions)
    "a": (dict(vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, intermediate_size=128, rms_norm_eps=1e-6, rope_theta=10000.0,
               tie_word_embeddings=True), 11, 33, (5, 3, 24, 1)),
    "b": (dict(vocab_size=512, hidden_size=192, num_hidden_layers=3, num_attention_heads=6,
               num_key_value_heads=3, intermediate_size=320, rms_norm_eps=1e-5, rope_theta=1000000.0,
               tie_word_embeddings=False), 12, 40, (7, 2, 13, 3, 2, 13)),
}


def main(ref_root):
    if sys.flags.optimize == 0:
        sys.exit(subprocess.call([sys.executable, "-O", os.path.abspath(__file__), ref_root]))
    sys.path.insert(0, os.path.join(ref_root, "pico_vllm"))
    sys.path.insert(0, os.path.join(ref_root, "pico_vllm", "legacy"))
    sys.path.insert(0, os.path.dirname(HERE))
    import torch
    from safetensors.torch import save_file
    import plain_qwen2 as plain
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "legacy_model", os.path.join(ref_root, "pico_vllm", "legacy", "model.py"))
    legacy = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(legacy)
    from cache import NaiveKVCache

    out = {}
    for name, (kw, seed, n_prompt, portions) in CASES.items():
        cfg = plain.config_dict(**kw)
        w = plain.random_weights(cfg, seed)
        mcfg = legacy.ModelConfig(
            vocab_size=kw["vocab_size"], hidden_size=kw["hidden_size"],
            num_hidden_layers=kw["num_hidden_layers"], num_attention_heads=kw["num_attention_heads"],
            num_key_value_heads=kw["num_key_value_heads"], intermediate_size=kw["intermediate_size"],
            rms_norm_eps=kw["rms_norm_eps"], rope_theta=kw["rope_theta"],
            tie_word_embeddings=kw["tie_word_embeddings"])
        model = legacy.Qwen25_15B(mcfg).float().eval()
        sd = {}
        for k, v in w.items():
            k = k.replace("model.", "", 1) if k.startswith("model.") else k
            k = (k.replace("self_attn.", "attn.").replace("mlp.", "ffn.")
                 .replace("input_layernorm", "norm1").replace("post_attention_layernorm", "norm2"))
            sd[k] = v
        missing, unexpected = model.load_state_dict(sd, strict=False)
        assert not unexpected, unexpected
        assert all("rope" in m for m in missing), missing
        g = torch.Generator().manual_seed(seed + 100)
        ids = torch.randint(0, kw["vocab_size"], (n_prompt,), generator=g)

        def cache():
            return NaiveKVCache(mcfg.num_hidden_layers, 64, mcfg.num_key_value_heads, mcfg.head_dim,
                                "cpu", torch.float32)
        with torch.no_grad():
            whole = model(ids[None, :], cache())[0]
            c = cache()
            parts, at = [], 0
            assert sum(portions) == n_prompt
            for n in portions:
                parts.append(model(ids[None, at:at + n], c)[0])
                at += n
            cut = torch.cat(parts, dim=0)
        out[f"{name}.ids"] = ids.to(torch.int32)
        out[f"{name}.logits_whole"] = whole.contiguous()
        out[f"{name}.logits_portions"] = cut.contiguous()
        print(name, "whole vs portions max abs diff", float((whole - cut).abs().max()))
    save_file(out, os.path.join(HERE, "legacy_tiny.safetensors"))
    print("wrote", os.path.join(HERE, "legacy_tiny.safetensors"))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py REFERENCE_CHECKOUT")
    main(sys.argv[1])
