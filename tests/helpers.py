"""Shared by the tests: the tiny configurations, model folders, and the four ways of
cutting requests into steps."""
import json
import os

import torch

import plain_qwen2 as plain

# Two tiny configurations that differ in every size and option.
TINY = {
    # A: 2 layers, width 64, 4 heads on 2 kv heads of 16, tied head, no window, page 16
    "a": dict(raw=dict(architectures=["Qwen2ForCausalLM"], vocab_size=256, hidden_size=64, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, intermediate_size=128, rope_theta=10000.0,
                       rms_norm_eps=1e-6, tie_word_embeddings=True, use_sliding_window=False,
                       max_position_embeddings=2048),
              page_size=16, seed=101),
    # B: 3 layers, width 192, 6 heads on 3 kv heads of 32 (sizes that are no power of two), untied head, page 8, and - so that the
    # two differ in every option - a window of 24 keys in the layers from index 1 on
    "b": dict(raw=dict(architectures=["Qwen2ForCausalLM"], vocab_size=512, hidden_size=192, num_hidden_layers=3,
                       num_attention_heads=6, num_key_value_heads=3, intermediate_size=320, rope_theta=1000000.0,
                       rms_norm_eps=1e-5, tie_word_embeddings=False, use_sliding_window=True, sliding_window=24,
                       max_window_layers=1, max_position_embeddings=4096),
              page_size=8, seed=202),
    # C: odd head size (48 = 3 x 16) with an explicit head_dim, one kv head, 5 query heads, odd vocabulary
    "c": dict(raw=dict(architectures=["Qwen2ForCausalLM"], vocab_size=331, hidden_size=80, num_hidden_layers=2,
                       num_attention_heads=5, num_key_value_heads=1, head_dim=48, intermediate_size=176,
                       rope_theta=50000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
                       max_position_embeddings=1024),
              page_size=4, seed=303),
    # D and E: the head sizes of the served models (64 and 128), which the TMA decode kernel and the tcgen05
    # prefill kernel take; D with a window in its second layer, E with three query heads on one kv head
    "d": dict(raw=dict(architectures=["Qwen2ForCausalLM"], vocab_size=300, hidden_size=256, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, intermediate_size=384, rope_theta=1000000.0,
                       rms_norm_eps=1e-6, tie_word_embeddings=True, use_sliding_window=True, sliding_window=40,
                       max_window_layers=1, max_position_embeddings=4096),
              page_size=16, seed=404),
    "e": dict(raw=dict(architectures=["Qwen2ForCausalLM"], vocab_size=411, hidden_size=192, num_hidden_layers=2,
                       num_attention_heads=3, num_key_value_heads=1, head_dim=128, intermediate_size=272,
                       rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                       max_position_embeddings=2048),
              page_size=32, seed=505),
    # F: width 2048 (16 query heads on 2 kv heads of 128): wider than the rows the fused norm keeps in registers
    "f": dict(raw=dict(architectures=["Qwen2ForCausalLM"], vocab_size=350, hidden_size=2048, num_hidden_layers=2,
                       num_attention_heads=16, num_key_value_heads=2, intermediate_size=384, rope_theta=1000000.0,
                       rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=2048),
              page_size=16, seed=606),
}


def tiny_config(name):
    from pico_vllm_b200.registry import config_from_dict
    return config_from_dict(TINY[name]["raw"])


def plain_config(cfg):
    return plain.config_dict(cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads,
                             cfg.num_key_value_heads, cfg.intermediate_size, cfg.rms_norm_eps, cfg.rope_theta,
                             cfg.tie_word_embeddings, head_dim=cfg.head_dim, layer_windows=list(cfg.layer_windows))


def tiny_tensors(name, dtype=torch.float32):
    from pico_vllm_b200.weights import random_tensors
    return random_tensors(tiny_config(name), TINY[name]["seed"], dtype=dtype)


def write_tiny_model(name, folder, dtype="bfloat16"):
    from pico_vllm_b200.weights import write_random_model
    return write_random_model(tiny_config(name), TINY[name]["seed"], str(folder), dtype=dtype)


def random_ids(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ------------------------------------------------------------------ ways of cutting requests into steps
def trace_whole(requests):
    """Each request alone and whole, one step each; logits wanted everywhere."""
    steps = []
    for rid, ids in requests.items():
        steps.append(dict(entries=[dict(id=rid, tokens=ids, want=list(range(len(ids))))], end=[rid]))
    return steps


def trace_tail_decode(requests, tail=32):
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append(dict(entries=[dict(id=rid, tokens=ids[:head], want=list(range(head)))], end=[]))
        for i in range(head, len(ids)):
            steps.append(dict(entries=[dict(id=rid, tokens=[ids[i]], want=[0])],
                              end=[rid] if i == len(ids) - 1 else []))
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests, sizes=(7, 2, 13, 3, 2, 29, 5, 2, 64, 11)):
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, ids in requests.items():
        at, k = 0, 0
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            if len(ids) - at - n == 1:     # never leave a single token for last unless unavoidable
                n += 1
            last = at + n >= len(ids)
            steps.append(dict(entries=[dict(id=rid, tokens=ids[at:at + n], want=list(range(n)))],
                              end=[rid] if last else []))
            at += n
            k += 1
    return steps


def trace_mixed(requests, max_live=4, seed=0, chunk_sizes=(5, 17, 2, 9, 33, 3)):
    """Up to ``max_live`` requests at a time: each first runs most of its tokens as portions of
    changing size, then its last tokens one by one, while others are at other stages; a request
    is sometimes left out of a step.  New requests start as old ones end, so pages are reused."""
    import random
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}       # rid -> [ids, next position, decode_from]
    steps = []
    k = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting.pop(0)
            live[rid] = [ids, 0, max(1, len(ids) - rng.choice([3, 8, 20]))]
        entries, end = [], []
        for rid in list(live):
            ids, at, dec = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                     # left out of this step
            if at < dec:
                n = min(chunk_sizes[k % len(chunk_sizes)], dec - at)
                k += 1
            else:
                n = 1
            entries.append(dict(id=rid, tokens=ids[at:at + n], want=list(range(n))))
            live[rid][1] = at + n
            if at + n >= len(ids):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append(dict(entries=entries, end=end))
    return steps


def trace_many_decoders(requests, tail=6, per_step=8, want_every=3):
    """Many requests live at once: all but the last ``tail`` tokens of each as whole prompts, ``per_step``
    requests a step; then ``tail`` steps that hold one token of every request, of which only every
    ``want_every``-th row (another set each step) is wanted."""
    rids = list(requests)
    steps = []
    for at in range(0, len(rids), per_step):
        entries = []
        for rid in rids[at:at + per_step]:
            head = requests[rid][:-tail]
            entries.append(dict(id=rid, tokens=head, want=[len(head) - 1]))
        steps.append(dict(entries=entries, end=[]))
    for k in range(tail):
        entries = []
        for j, rid in enumerate(rids):
            ids = requests[rid]
            entries.append(dict(id=rid, tokens=[ids[len(ids) - tail + k]], want=[0] if (j + k) % want_every == 0 else []))
        steps.append(dict(entries=entries, end=rids if k == tail - 1 else []))
    return steps


def live_token_peak(steps, round_to=64):
    """Most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def expected_logits(steps, requests, plain_logits):
    """For every step, the plain implementation's logits at the wanted places ([wanted, vocab])."""
    at = {rid: 0 for rid in requests}
    out = []
    for st in steps:
        rows = []
        for e in st["entries"]:
            rid = e["id"]
            for w in e["want"]:
                rows.append(plain_logits[rid][at[rid] + w])
            at[rid] += len(e["tokens"])
        for rid in st["end"]:
            at[rid] = 0
        out.append(torch.stack(rows) if rows else None)
    return out


def replay(runner, steps):
    """Drives a ModelRunner like bin/trace_run does; returns the logits of every step (or None)."""
    from pico_vllm_b200.engine import StepItem
    slots, out = {}, []
    for st in steps:
        items = []
        for e in st["entries"]:
            if e["id"] not in slots:
                slots[e["id"]] = runner.cache.acquire(e["id"])
            items.append(StepItem(slots[e["id"]], e["tokens"], tuple(e["want"])))
        logits = runner.step(items)
        out.append(logits.detach().float().cpu().clone() if logits.shape[0] else None)
        for rid in st["end"]:
            runner.cache.release(slots.pop(rid))
        runner.cache.check()
    return out


def make_runner_from_tensors(name, dtype, device, max_tokens, max_num_seqs=4, use_cuda_graph=False,
                             poison=True, page_size=None, **options):
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine import ModelRunner, make_cache, model_from_tensors
    cfg = tiny_config(name)
    ecfg = EngineConfig(dtype=dtype, page_size=page_size or TINY[name]["page_size"], max_cache_tokens=max_tokens,
                        max_num_seqs=max_num_seqs, use_cuda_graph=use_cuda_graph, device=device, **options)
    tensors = tiny_tensors(name, torch.float32 if dtype == "float32" else torch.bfloat16)
    model = model_from_tensors(cfg, tensors, ecfg)
    return ModelRunner(model, make_cache(model, ecfg, poison_freed=poison), ecfg), tensors


def assert_close_logits(got, want, rel, what=""):
    """max |got - want| <= rel * max |want| over the whole step."""
    scale = float(want.abs().max())
    err = float((got.double() - want.double()).abs().max())
    assert err <= rel * scale, f"{what}: max abs error {err:.3e} > {rel:g} * {scale:.3e}"
