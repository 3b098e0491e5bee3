"""The whole model at the layer sizes that are served and benchmarked (width 1536, 12 query heads
on 2 key/value heads of 128, feed-forward 8960, vocabulary 151936, tied head), cut to 2 or 4
layers, against the plain implementation: every way of cutting requests into steps, in 32-bit
and in bfloat16, with graph replay on and off.  These sizes reach the kernels that the tiny
configurations do not: the products with the norm inside at K = 1536, the paired-SM gate_up
product from 200 tokens on, prompt attention over several 128-row tiles, a portion late in a
long context (two blocks per query tile), split decode attention with six query heads per kv
head, and the 151936-row head.

The reference's nearest check is the float32 model-against-oracle logit comparison in
pico_vllm/legacy/model.py:229-289; its engine test compares generated text
(pico_vllm/tests/test_engine.py:59-93).

The vocabulary is too large to keep logits of every position, so the plain implementation's
states before the head are kept and its head is applied to the wanted rows only.
"""
import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
REL = {"float32": 5e-5, "bfloat16": 3e-2}     # max |difference| / max |logit| over a step
RAW = dict(architectures=["Qwen2ForCausalLM"], vocab_size=151936, hidden_size=1536, num_hidden_layers=4,
           num_attention_heads=12, num_key_value_heads=2, intermediate_size=8960, rope_theta=1000000.0,
           rms_norm_eps=1e-6, tie_word_embeddings=True, use_sliding_window=False, max_position_embeddings=32768)
SEED = 1536
LENGTHS = [760, 300, 150, 90, 41]

_cache = {}


def _config(layers):
    from pico_vllm_b200.registry import config_from_dict
    return config_from_dict(dict(RAW, num_hidden_layers=layers))


def _tensors(layers, dtype):
    """Float32 draws of the 4-layer model, once; fewer layers take the first ones; bfloat16 is their rounding."""
    from pico_vllm_b200.weights import random_tensors
    if "f32" not in _cache:
        _cache["f32"] = random_tensors(_config(4), SEED, dtype=torch.float32)
    key = (layers, dtype)
    if key not in _cache:
        keep = {n: t for n, t in _cache["f32"].items()
                if not n.startswith("model.layers.") or int(n.split(".")[2]) < layers}
        _cache[key] = keep if dtype == "float32" else {n: t.to(torch.bfloat16) for n, t in keep.items()}
    return _cache[key]


class PlainRows:
    """Row p = the plain implementation's logits at position p, computed when asked for."""

    def __init__(self, ids, tensors, pcfg):
        self.w = {"model.embed_tokens.weight": tensors["model.embed_tokens.weight"].float()}
        self.pcfg = pcfg
        self.states = plain.last_hidden_states(ids, tensors, pcfg)
        self.rows = {}

    def __getitem__(self, p):
        if p not in self.rows:
            self.rows[p] = plain.lm_head(self.states[p:p + 1], self.w, self.pcfg)[0]
        return self.rows[p]


def _plain(layers, dtype, reqs):
    out = {}
    for rid, ids in reqs.items():
        key = ("plain", layers, dtype, rid, len(ids))
        if key not in _cache:
            _cache[key] = PlainRows(ids, _tensors(layers, dtype), helpers.plain_config(_config(layers)))
        out[rid] = _cache[key]
    return out


def _requests(lengths=LENGTHS):
    return {f"r{i}": helpers.random_ids(n, RAW["vocab_size"], 4000 + i) for i, n in enumerate(lengths)}


def _thin(steps, every=13):
    """Fewer wanted rows in portions (the first, the last and every 13th); single tokens keep theirs."""
    for st in steps:
        for e in st["entries"]:
            n = len(e["tokens"])
            if n > 2:
                e["want"] = sorted({0, n - 1} | set(range(0, n, every)))
    return steps


def _runner(layers, dtype, max_tokens, graph, max_num_seqs=4, **options):
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine import ModelRunner, make_cache, model_from_tensors
    key = ("model", layers, dtype)
    ecfg = EngineConfig(dtype=dtype, page_size=16, max_cache_tokens=max_tokens, max_num_seqs=max_num_seqs,
                        use_cuda_graph=graph, device=DEV, **options)
    if key not in _cache:
        for k in [k for k in _cache if k[0] == "model"]:
            del _cache[k]                      # one model on the device at a time
        _cache[key] = model_from_tensors(_config(layers), _tensors(layers, dtype), ecfg)
    model = _cache[key]
    return ModelRunner(model, make_cache(model, ecfg, poison_freed=True), ecfg)


def _compare(runner, steps, reqs, plain_rows, dtype, what):
    from pico_vllm_b200 import ops
    want = helpers.expected_logits(steps, reqs, plain_rows)
    got = helpers.replay(runner, steps)
    for i, (g, w) in enumerate(zip(got, want)):
        assert (g is None) == (w is None), f"{what} step {i}"
        if w is not None:
            assert torch.isfinite(g).all(), f"{what} step {i}: not finite (a freed page was read?)"
            helpers.assert_close_logits(g, w, REL[dtype], f"{what} step {i}")
    assert all(g.pool.in_use == 0 for g in runner.cache.groups)
    assert ops.tc_status() == 0 and ops.tca_status() == 0 and ops.tma_status() == 0


_CUTS = {
    "whole": helpers.trace_whole,
    "tail": lambda r: helpers.trace_tail_decode(r, 32),
    "portions": lambda r: helpers.trace_portions(r, (7, 2, 210, 13, 3, 2, 129, 29, 5, 2, 64, 11)),
    "mixed": lambda r: helpers.trace_mixed(r, max_live=4, seed=3, chunk_sizes=(5, 217, 2, 9, 33, 3, 140)),
}


@pytest.mark.parametrize("cut,graph", [("whole", False), ("tail", False), ("tail", True), ("portions", False),
                                       ("mixed", False), ("mixed", True)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])       # the slowest-changing: one model upload per dtype
def test_real_layer_sizes_every_cutting_matches_plain(dtype, cut, graph):
    reqs = _requests()
    steps = _thin(_CUTS[cut](reqs))
    runner = _runner(2, dtype, helpers.live_token_peak(steps), graph)
    _compare(runner, steps, reqs, _plain(2, dtype, reqs), dtype, f"2 layers/{cut}/{dtype}/graph={graph}")
    if graph:
        assert runner.graph_replays > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_four_layers_mixed(dtype):
    """Four layers, so that a layer's cache entry taken for another's would show."""
    reqs = _requests([333, 140, 77, 30])
    steps = _thin(helpers.trace_mixed(reqs, max_live=4, seed=8, chunk_sizes=(5, 217, 2, 9, 33, 3)))
    runner = _runner(4, dtype, helpers.live_token_peak(steps), True)
    _compare(runner, steps, reqs, _plain(4, dtype, reqs), dtype, f"4 layers/mixed/{dtype}")


def test_real_layer_sizes_a_portion_late_in_a_long_context():
    """bfloat16: three full portions of 2,048 tokens replayed from the prompt graph, a fourth after
    6,144 tokens (where prompt attention gives every query tile two blocks, at the default
    ``pair_min_context``), a short last portion, then 24 tokens one by one at a context of 8,300
    (16-way split decode attention)."""
    dtype = "bfloat16"
    P = 2048
    reqs = _requests([4 * P + 77 + 24])
    ids = reqs["r0"]
    steps = []
    for k in range(4):
        steps.append(dict(entries=[dict(id="r0", tokens=ids[k * P:(k + 1) * P], want=[P - 1])], end=[]))
    steps[3]["entries"][0]["want"] = [0, 1, 500, 1023, 1024, 2000, P - 1]       # more rows only when launched directly
    steps.append(dict(entries=[dict(id="r0", tokens=ids[4 * P:4 * P + 77], want=[0, 40, 76])], end=[]))
    for i in range(4 * P + 77, len(ids)):
        steps.append(dict(entries=[dict(id="r0", tokens=[ids[i]], want=[0])], end=["r0"] if i == len(ids) - 1 else []))
    runner = _runner(2, dtype, helpers.live_token_peak(steps), True, max_num_batched_tokens=P)
    assert runner.cfg.pair_min_context == 6144
    _compare(runner, steps, reqs, _plain(2, dtype, reqs), dtype, "2 layers/long context/bfloat16")
    assert runner.graph_replays >= 3 + 24


@pytest.mark.parametrize("dtype,live,graph", [("float32", 20, True), ("bfloat16", 5, True), ("bfloat16", 33, False),
                                              ("bfloat16", 33, True), ("bfloat16", 64, True)])
def test_real_layer_sizes_decode_steps_of_many_live_requests(dtype, live, graph):
    """Decode-only steps of 5 to 64 requests at the served layer sizes: 8 parts of the key range per token at
    5 requests, fewer as the batch grows; the products for more than 16 tokens; graph buckets 8, 32 and 64; logits
    of only some rows."""
    # one long request sets the number of parts (the step's longest context decides); the others are short
    reqs = {f"d{i}": helpers.random_ids(1100 if i == 0 else 30 + (i * 37) % 60, RAW["vocab_size"], 7000 + i)
            for i in range(live)}
    steps = helpers.trace_many_decoders(reqs, tail=4, per_step=8)
    runner = _runner(2, dtype, helpers.live_token_peak(steps), graph, max_num_seqs=64, max_num_batched_tokens=4096)
    _compare(runner, steps, reqs, _plain(2, dtype, reqs), dtype, f"2 layers/{live} live/{dtype}/graph={graph}")
    if graph:
        assert runner.graph_replays == 4
