"""The plain implementation against the reference's own pure-torch model (stored outputs)
and against itself in float64."""
import os

import pytest
import torch
from safetensors.torch import load_file

import plain_qwen2 as plain
from golden.make_golden import CASES

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "legacy_tiny.safetensors")


@pytest.mark.parametrize("name", sorted(CASES))
def test_plain_equals_reference_legacy_model(name):
    kw, seed, n_prompt, _ = CASES[name]
    gold = load_file(GOLDEN)
    cfg = plain.config_dict(**kw)
    w = plain.random_weights(cfg, seed)
    ids = gold[f"{name}.ids"].long()
    assert ids.shape[0] == n_prompt
    mine = plain.forward(ids, w, cfg)
    for key in ("logits_whole", "logits_portions"):
        ref = gold[f"{name}.{key}"]
        scale = float(ref.abs().max())
        assert float((mine - ref).abs().max()) <= 2e-5 * scale, key


def test_plain_float64_agrees_with_float32():
    kw, seed, _, _ = CASES["b"]
    cfg = plain.config_dict(**kw)
    w = plain.random_weights(cfg, seed)
    ids = torch.arange(0, 30) * 7 % kw["vocab_size"]
    a = plain.forward(ids, w, cfg, torch.float32)
    b = plain.forward(ids, w, cfg, torch.float64)
    assert float((a.double() - b).abs().max()) <= 1e-5 * float(b.abs().max())


def test_window_hides_far_keys():
    # one query whose best key lies outside the window must not see it
    T, hd = 12, 16
    q = torch.zeros(T, 1, hd)
    k = torch.zeros(T, 1, hd)
    v = torch.arange(T, dtype=torch.float32)[:, None, None].expand(T, 1, hd).clone()
    q[-1, 0, 0] = 50.0
    k[2, 0, 0] = 50.0            # a far key with a huge score
    pos = torch.arange(T)
    full = plain.attention_scores_softmax_pv(q, k, v, pos, None)
    win = plain.attention_scores_softmax_pv(q, k, v, pos, 4)
    assert abs(float(full[-1, 0, 0]) - 2.0) < 1e-3
    assert abs(float(win[-1, 0, 0]) - (8 + 9 + 10 + 11) / 4) < 1e-4


def test_prefix_of_a_sequence_has_the_same_logits():
    kw, seed, _, _ = CASES["a"]
    cfg = plain.config_dict(**kw)
    w = plain.random_weights(cfg, seed)
    ids = torch.arange(0, 20) * 5 % kw["vocab_size"]
    whole = plain.forward(ids, w, cfg)
    part = plain.forward(ids[:11], w, cfg)
    assert torch.allclose(whole[:11], part, atol=1e-6)


def test_top_p_filter_keeps_the_smallest_set():
    probs = torch.tensor([[0.1, 0.5, 0.15, 0.25]])
    out = plain.top_p_filter(probs, 0.7)
    assert torch.allclose(out, torch.tensor([[0.0, 0.5 / 0.75, 0.0, 0.25 / 0.75]]))
