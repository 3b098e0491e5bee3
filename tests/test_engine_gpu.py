"""The engine on the GPU against the plain implementation, in 32-bit and in bfloat16: every
way of cutting requests into steps, long decoding, first tokens, generation through the entry
point, graph replay, parts alone, and toy parts defined here (a mixer with state of its own, a
feed-forward with routing, another position encoding)."""
import math

import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
REL = {"float32": 5e-5, "bfloat16": 3e-2}     # max |difference| / max |logit| over a step
LENGTHS = {"a": [5, 17, 33, 70, 150], "b": [1, 9, 24, 40, 77, 131], "c": [3, 21, 50, 97],
           "d": [4, 30, 66, 129, 200], "e": [2, 19, 65, 140]}


def _requests(name, vocab):
    return {f"r{i}": helpers.random_ids(n, vocab, 1000 + i) for i, n in enumerate(LENGTHS[name])}


def _plain_logits(name, reqs, tensors):
    cfg = helpers.tiny_config(name)
    return {rid: plain.forward(ids, tensors, helpers.plain_config(cfg)) for rid, ids in reqs.items()}


_CUTS = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_tail_decode(r, 32),
         "portions": helpers.trace_portions, "mixed": helpers.trace_mixed}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("graph", [False, True])
def test_every_cutting_matches_plain(dtype, name, cut, graph):
    if graph and cut in ("whole", "portions"):
        pytest.skip("no single-token steps in this cutting")
    cfg = helpers.tiny_config(name)
    reqs = _requests(name, cfg.vocab_size)
    steps = _CUTS[cut](reqs)
    runner, tensors = helpers.make_runner_from_tensors(name, dtype, DEV, helpers.live_token_peak(steps),
                                                       use_cuda_graph=graph)
    want = helpers.expected_logits(steps, reqs, _plain_logits(name, reqs, tensors))
    got = helpers.replay(runner, steps)
    for i, (g, w) in enumerate(zip(got, want)):
        assert (g is None) == (w is None)
        if w is not None:
            assert torch.isfinite(g).all(), f"{name}/{cut} step {i}: not finite (a freed page was read?)"
            helpers.assert_close_logits(g, w, REL[dtype], f"{name}/{cut}/{dtype} step {i}")
    if graph:
        assert runner.graph_replays > 0
    assert all(g.pool.in_use == 0 for g in runner.cache.groups)


@pytest.mark.parametrize("graph", [False, True])
def test_greedy_tokens_chosen_inside_the_head_are_the_argmax_of_its_logits(graph):
    """``step(..., greedy=True)`` leaves the tokens in ``runner.feedback`` and writes no logits where the head's
    kernel can choose them (bfloat16, up to 16 wanted rows, a vocabulary that is a multiple of 16): the same steps
    through a second runner with logits must give the same tokens, for decode steps (recorded and replayed),
    a mixed step, and a step where not every row is wanted."""
    from pico_vllm_b200.engine import StepItem
    name = "a"
    cfg = helpers.tiny_config(name)
    ra, _ = helpers.make_runner_from_tensors(name, "bfloat16", DEV, 512, max_num_seqs=8, use_cuda_graph=graph)
    rb, _ = helpers.make_runner_from_tensors(name, "bfloat16", DEV, 512, max_num_seqs=8, use_cuda_graph=graph)
    prompts = [helpers.random_ids(n, cfg.vocab_size, 700 + n) for n in (9, 30, 4, 17, 22)]
    sa = [ra.cache.acquire(i) for i in range(5)]
    sb = [rb.cache.acquire(i) for i in range(5)]
    # a mixed step: three prompts whole, rows wanted at their ends
    items = lambda slots, toks, want: [StepItem(s, t, w) for s, t, w in zip(slots, toks, want)]
    want = [(len(p) - 1,) for p in prompts[:3]]
    assert ra.step(items(sa[:3], prompts[:3], want), greedy=True) is None
    logits = rb.step(items(sb[:3], prompts[:3], want))
    last = logits.argmax(-1).tolist()
    assert ra.feedback[:3].tolist() == last
    for k in range(6):                              # decode steps: 3, then 5 requests (two join with their prompts first)
        if k == 2:
            w2 = [(len(p) - 1,) for p in prompts[3:]]
            assert ra.step(items(sa[3:], prompts[3:], w2), greedy=True) is None
            last += rb.step(items(sb[3:], prompts[3:], w2)).argmax(-1).tolist()
            assert ra.feedback[:2].tolist() == last[3:]
        n = len(last)
        toks = [[t] for t in last]
        out = ra.step(items(sa[:n], toks, [(0,)] * n), greedy=True)
        assert out is None
        last = rb.step(items(sb[:n], toks, [(0,)] * n)).argmax(-1).tolist()
        assert ra.feedback[:n].tolist() == last, f"decode step {k}"
    # not every row wanted: tokens of the wanted rows, in order (a recorded step computes every row of its
    # bucket, so there logits come back instead, for the wanted rows only)
    n = len(last)
    out = ra.step(items(sa[:n], [[t] for t in last], [(0,), (), (0,), (), (0,)]), greedy=True)
    ref = rb.step(items(sb[:n], [[t] for t in last], [(0,), (), (0,), (), (0,)]))
    assert ref.shape == (3, cfg.vocab_size)
    if graph:
        assert out is not None and out.shape == ref.shape and torch.equal(out.argmax(-1), ref.argmax(-1))
    else:
        assert out is None and ra.feedback[:3].tolist() == ref.argmax(-1).tolist()
    if graph:
        assert ra.graph_replays >= 6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", ["tail", "mixed"])
def test_a_model_2048_wide(dtype, cut):
    """Width 2048 (the next larger served shape): at up to 8 tokens the fused norm reads its rows twice instead
    of keeping them in registers; from 9 tokens on the norm is a kernel of its own."""
    cfg = helpers.tiny_config("f")
    reqs = {f"r{i}": helpers.random_ids(n, cfg.vocab_size, 2000 + i) for i, n in enumerate([70, 33, 150, 12, 40, 25])}
    steps = (helpers.trace_tail_decode(reqs, 12) if cut == "tail"
             else helpers.trace_many_decoders(reqs, tail=5, per_step=3, want_every=2))
    runner, tensors = helpers.make_runner_from_tensors("f", dtype, DEV, helpers.live_token_peak(steps), max_num_seqs=8,
                                                       use_cuda_graph=(cut == "mixed"))
    want = helpers.expected_logits(steps, reqs, _plain_logits("f", reqs, tensors))
    for i, (g, w) in enumerate(zip(helpers.replay(runner, steps), want)):
        if w is not None:
            helpers.assert_close_logits(g, w, REL[dtype], f"f/{cut}/{dtype} step {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["d", "e"])
@pytest.mark.parametrize("live", [5, 20, 33, 64])
@pytest.mark.parametrize("graph", [False, True])
def test_decode_steps_of_many_live_requests(dtype, name, live, graph):
    """Decode-only steps of 5 to 64 requests: the graph buckets 8 to 64 (padded), the products for more than
    16 tokens in a decode step, fewer splits of the key range as the batch grows, and logits of only some rows."""
    cfg = helpers.tiny_config(name)
    reqs = {f"r{i}": helpers.random_ids(9 + (i * 7) % 45, cfg.vocab_size, 300 + i) for i in range(live)}
    steps = helpers.trace_many_decoders(reqs)
    runner, tensors = helpers.make_runner_from_tensors(name, dtype, DEV, helpers.live_token_peak(steps),
                                                       max_num_seqs=64, use_cuda_graph=graph,
                                                       max_num_batched_tokens=4096)
    want = helpers.expected_logits(steps, reqs, _plain_logits(name, reqs, tensors))
    got = helpers.replay(runner, steps)
    for i, (g, w) in enumerate(zip(got, want)):
        assert (g is None) == (w is None)
        if w is not None:
            assert g.shape == w.shape
            helpers.assert_close_logits(g, w, REL[dtype], f"{name}/{dtype}/{live} live step {i}")
    if graph:
        assert runner.graph_replays == 6
    assert all(g.pool.in_use == 0 for g in runner.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["b", "d", "e"])
@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_cuttings_match_plain(dtype, name, seed):
    """Random requests, cut at random: portions of 2 to 40 tokens or single tokens, up to four live, requests left
    out of steps at random, graph replay on, a pool of exactly the live peak (pages come back and are used again)."""
    import random
    rng = random.Random(seed)
    cfg = helpers.tiny_config(name)
    reqs = {f"r{i}": helpers.random_ids(rng.randint(2, 180), cfg.vocab_size, 5000 + 10 * seed + i) for i in range(7)}
    sizes = tuple(rng.choice([2, 3, 5, 8, 13, 21, 40]) for _ in range(9))
    steps = helpers.trace_mixed(reqs, max_live=rng.randint(2, 4), seed=seed, chunk_sizes=sizes)
    runner, tensors = helpers.make_runner_from_tensors(name, dtype, DEV, helpers.live_token_peak(steps), use_cuda_graph=True)
    want = helpers.expected_logits(steps, reqs, _plain_logits(name, reqs, tensors))
    for i, (g, w) in enumerate(zip(helpers.replay(runner, steps), want)):
        if w is not None:
            assert torch.isfinite(g).all(), f"step {i}: not finite (a freed page was read?)"
            helpers.assert_close_logits(g, w, REL[dtype], f"{name}/{dtype}/seed {seed} step {i}")
    assert all(g.pool.in_use == 0 for g in runner.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "d"])
def test_long_decoding(dtype, name):
    """A short prompt, then 400 tokens one by one (pages fill up, the window moves on)."""
    cfg = helpers.tiny_config(name)
    ids = helpers.random_ids(420, cfg.vocab_size, 77)
    reqs = {"x": ids}
    steps = helpers.trace_tail_decode(reqs, 400)
    runner, tensors = helpers.make_runner_from_tensors(name, dtype, DEV, 448, use_cuda_graph=True)
    want = helpers.expected_logits(steps, reqs, _plain_logits(name, reqs, tensors))
    got = helpers.replay(runner, steps)
    for i, (g, w) in enumerate(zip(got, want)):
        helpers.assert_close_logits(g, w, REL[dtype], f"{name}/{dtype} step {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "d", "e"])
def test_long_prompts_in_one_step(dtype, name):
    """Prompts of several hundred tokens, whole and as two requests in one step: in bfloat16 these
    sizes go through the tcgen05 kernels (gate_up products on pairs of SMs from 200 tokens on,
    attention tiles of 128 rows with several key tiles)."""
    cfg = helpers.tiny_config(name)
    reqs = {"x": helpers.random_ids(700, cfg.vocab_size, 31), "y": helpers.random_ids(300, cfg.vocab_size, 32)}
    steps = [dict(entries=[dict(id="x", tokens=reqs["x"], want=list(range(0, 700, 7)))], end=["x"]),
             dict(entries=[dict(id="x", tokens=reqs["x"][:450], want=[0, 449]),
                           dict(id="y", tokens=reqs["y"], want=list(range(0, 300, 3)))], end=["y"]),
             dict(entries=[dict(id="x", tokens=reqs["x"][450:], want=list(range(0, 250, 5)))], end=["x"])]
    runner, tensors = helpers.make_runner_from_tensors(name, dtype, DEV, 1100)
    want = helpers.expected_logits(steps, reqs, _plain_logits(name, reqs, tensors))
    for i, (g, w) in enumerate(zip(helpers.replay(runner, steps), want)):
        assert torch.isfinite(g).all()
        helpers.assert_close_logits(g, w, REL[dtype], f"{name}/{dtype} step {i}")
    from pico_vllm_b200 import ops
    assert ops.tc_status() == 0 and ops.tca_status() == 0 and ops.tma_status() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(dtype):
    """Position 0 alone, then 1, 2, 3 one by one: the shortest contexts."""
    cfg = helpers.tiny_config("c")
    reqs = {"x": helpers.random_ids(6, cfg.vocab_size, 5)}
    steps = helpers.trace_tail_decode(reqs, 5)
    runner, tensors = helpers.make_runner_from_tensors("c", dtype, DEV, 64)
    want = helpers.expected_logits(steps, reqs, _plain_logits("c", reqs, tensors))
    for i, (g, w) in enumerate(zip(helpers.replay(runner, steps), want)):
        helpers.assert_close_logits(g, w, REL[dtype], f"step {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_key_among_hundreds_and_page_edges(dtype):
    """Weights are random, so a far key would hardly matter: instead the first layer's query and
    key projections are scaled up, which makes attention sharp and every key position count."""
    name = "a"
    cfg = helpers.tiny_config(name)
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine import ModelRunner, make_cache, model_from_tensors
    tensors = helpers.tiny_tensors(name, torch.float32 if dtype == "float32" else torch.bfloat16)
    for k in ("q_proj", "k_proj"):
        tensors[f"model.layers.0.self_attn.{k}.weight"] = tensors[f"model.layers.0.self_attn.{k}.weight"] * 12
        tensors[f"model.layers.0.self_attn.{k}.bias"] = tensors[f"model.layers.0.self_attn.{k}.bias"] * 12
    ecfg = EngineConfig(dtype=dtype, page_size=16, max_cache_tokens=640, max_num_seqs=2, use_cuda_graph=False,
                        device=DEV)
    model = model_from_tensors(cfg, tensors, ecfg)
    runner = ModelRunner(model, make_cache(model, ecfg, poison_freed=True), ecfg)
    reqs = {"x": helpers.random_ids(600, cfg.vocab_size, 9)}
    # portions that end exactly on, one before and one after page edges
    sizes = (16, 15, 1, 17, 31, 2, 48, 63, 65, 128, 2, 212)
    steps = helpers.trace_portions(reqs, sizes)
    want = helpers.expected_logits(steps, reqs, _plain_logits(name, reqs, tensors))
    for i, (g, w) in enumerate(zip(helpers.replay(runner, steps), want)):
        helpers.assert_close_logits(g, w, REL[dtype] * (1 if dtype == "float32" else 2), f"step {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dtype, tmp_path):
    from pico_vllm_b200 import LLM, SamplingParams
    name = "b"
    cfg = helpers.tiny_config(name)
    helpers.write_tiny_model(name, tmp_path, dtype=dtype)
    llm = LLM(str(tmp_path), dtype=dtype, device=DEV, page_size=8, num_pages=40, max_num_seqs=4,
              max_num_batched_tokens=32, prefill_chunk=7, max_model_len=128)
    prompts = [helpers.random_ids(n, cfg.vocab_size, 50 + n) for n in (1, 9, 24, 40, 13, 30)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True))
    tensors = helpers.tiny_tensors(name, torch.float32 if dtype == "float32" else torch.bfloat16)
    pcfg = helpers.plain_config(cfg)
    for p, o in zip(prompts, outs):
        if dtype == "float32":
            assert o.token_ids == plain.greedy_generate(p, tensors, pcfg, 12)
        else:
            # bfloat16 may pick another token where two logits are close: follow the engine's own
            # tokens and require that each was (nearly) the plain implementation's best
            ids = list(p) + o.token_ids
            logits = plain.forward(ids, tensors, pcfg)
            for j, tok in enumerate(o.token_ids):
                row = logits[len(p) + j - 1]
                assert float(row.max() - row[tok]) <= 3e-2 * float(row.abs().max())
    llm.cache.check()
    assert all(g.pool.in_use == 0 for g in llm.cache.groups)


def test_a_folder_stored_in_32_bit_served_in_bfloat16(tmp_path):
    """Matrices stored in float32 stay float32 (their products run in float32); the rest of the
    bfloat16 path is as usual."""
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine import make_runner
    name = "c"
    cfg = helpers.tiny_config(name)
    helpers.write_tiny_model(name, tmp_path, dtype="float32")
    runner = make_runner(str(tmp_path), EngineConfig(dtype="bfloat16", page_size=4, max_cache_tokens=256,
                                                     max_num_seqs=2, device=DEV), poison_freed=True)
    assert runner.model.blocks[0].mixer.qkv_weight.dtype == torch.float32
    reqs = {"x": helpers.random_ids(150, cfg.vocab_size, 3)}
    steps = helpers.trace_portions(reqs, (130, 2, 1, 17))
    tensors = helpers.tiny_tensors(name, torch.float32)
    want = helpers.expected_logits(steps, reqs, _plain_logits(name, reqs, tensors))
    for i, (g, w) in enumerate(zip(helpers.replay(runner, steps), want)):
        helpers.assert_close_logits(g, w, REL["bfloat16"], f"step {i}")


def test_command_line_generates(tmp_path, capsys):
    from pico_vllm_b200.cli import main
    helpers.write_tiny_model("a", tmp_path, dtype="float32")
    prompts = [[5, 17, 3], [9, 9]]
    rc = main(["run", "--model", str(tmp_path), "--dtype", "float32", "--prompt-ids", "5,17,3", "--prompt-ids", "9,9",
               "--max-new-tokens", "4", "--temperature", "0", "--num-gpu-blocks", "32", "--ignore-eos"])
    assert rc == 0
    lines = [l for l in capsys.readouterr().out.splitlines() if l.startswith("[")]
    assert len(lines) == 2
    printed = {int(l[1:l.index("]")]): [int(t) for t in l.split("] ")[1].split()] for l in lines}
    tensors = helpers.tiny_tensors("a", torch.float32)
    pcfg = helpers.plain_config(helpers.tiny_config("a"))
    for rid, p in enumerate(prompts):       # the reference prints prompt and generated tokens together
        assert printed[rid] == p + plain.greedy_generate(p, tensors, pcfg, 4)


@pytest.mark.parametrize("ahead", [True, False])
def test_generation_with_preemption_and_end_tokens(ahead, tmp_path):
    """So few pages that requests are pre-empted and recomputed, and an end token that some requests
    meet, one step ahead of the device and in turn: a request that was pre-empted, or that ended, while
    a step of its own was in flight must neither lose nor keep a token, and every page comes back."""
    from pico_vllm_b200 import LLM, SamplingParams
    name = "b"
    cfg = helpers.tiny_config(name)
    helpers.write_tiny_model(name, tmp_path, dtype="float32")
    tensors = helpers.tiny_tensors(name, torch.float32)
    pcfg = helpers.plain_config(cfg)
    prompts = [helpers.random_ids(n, cfg.vocab_size, 50 + n) for n in (1, 9, 24, 40, 13, 30, 6, 21, 35)]
    want = [plain.greedy_generate(p, tensors, pcfg, 10) for p in prompts]
    from collections import Counter
    # the end token: the one that most requests meet before their last token
    eos = Counter(t for w in want for t in set(w[:-1])).most_common(1)[0][0]
    llm = LLM(str(tmp_path), dtype="float32", device=DEV, page_size=8, num_pages=11, max_num_seqs=4,
              max_num_batched_tokens=16, prefill_chunk=7, max_model_len=112, async_scheduling=ahead)
    llm.scheduler.eos_token_id = eos
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=10))
    hit = 0
    for w, o in zip(want, outs):
        cut = w.index(eos) + 1 if eos in w else len(w)
        assert o.token_ids == w[:cut]
        assert o.finish_reason == ("eos" if eos in w else "length")
        hit += eos in w
    assert hit >= 1 and llm.scheduler.num_preemptions > 0
    llm.cache.check()
    assert all(g.pool.in_use == 0 for g in llm.cache.groups) and llm.cache.free_slots == llm.cache.max_num_seqs
    from pico_vllm_b200 import ops
    ops.check_kernel_status()


def test_sampling_through_the_entry_point_is_reproducible(tmp_path):
    from pico_vllm_b200 import LLM, SamplingParams
    helpers.write_tiny_model("a", tmp_path, dtype="float32")
    cfg = helpers.tiny_config("a")
    prompts = [helpers.random_ids(n, cfg.vocab_size, 90 + n) for n in (4, 11, 19)]
    sp = SamplingParams(temperature=0.8, top_p=0.95, max_new_tokens=8, seed=11, ignore_eos=True)
    a = LLM(str(tmp_path), dtype="float32", device=DEV, max_cache_tokens=512).generate(prompts, sp)
    llm2 = LLM(str(tmp_path), dtype="float32", device=DEV, max_cache_tokens=512, max_num_batched_tokens=5)
    b = [llm2.generate([p], sp)[0] for p in prompts]
    assert [o.token_ids for o in a] == [o.token_ids for o in b]
    assert len({tuple(o.token_ids) for o in a}) > 1


# ------------------------------------------------------------------ parts alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parts_alone(dtype):
    """Norm, feed-forward and attention parts, each built by itself with sizes of its own."""
    from pico_vllm_b200.parts import GQAAttention, GatedMLP, RMSNorm, Rotary, CacheView
    from pico_vllm_b200.engine.batch import Batch, GroupBatch
    g = torch.Generator().manual_seed(1)
    t = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    W, T = 72, 11
    # norm
    norm = RMSNorm(W, 1e-4)
    norm.materialize(DEV, dtype)
    norm.weight = (1 + 0.1 * torch.randn(W, generator=g)).to(DEV)
    x = torch.randn(T, W, generator=g)
    d = torch.randn(T, W, generator=g).to(dtype)
    xg = x.to(DEV)
    y = norm.add_norm(xg, d.to(DEV))
    want = plain.rms_norm(x + d.float(), norm.weight.cpu(), 1e-4)
    assert torch.allclose(y.cpu().float(), want, **t)
    # feed-forward
    mlp = GatedMLP(W, 100)
    wg, wu, wd = (torch.randn(100, W, generator=g) * 0.1, torch.randn(100, W, generator=g) * 0.1,
                  torch.randn(W, 100, generator=g) * 0.1)
    mlp.gate_up_weight = torch.cat([wg, wu]).to(dtype).to(DEV)
    mlp.down_weight = wd.to(dtype).to(DEV)
    h = torch.randn(T, W, generator=g).to(dtype)
    got = mlp.forward(h.to(DEV), None).cpu().float()
    w = {"gate_proj.weight": wg.to(dtype).float(), "up_proj.weight": wu.to(dtype).float(),
         "down_proj.weight": wd.to(dtype).float()}
    assert torch.allclose(got, plain.swiglu_mlp(h.float(), w, ""), **t)
    # attention: one request, 11 tokens at once, against the plain whole-sequence attention
    nh, nkv, hd, ps = 6, 2, 16, 4
    attn = GQAAttention(W, nh, nkv, hd, position=Rotary(hd, 777.0), window=5)
    attn.materialize(DEV, dtype)
    ws = {n: torch.randn(o, W, generator=g) * 0.2 for n, o in (("q", nh * hd), ("k", nkv * hd), ("v", nkv * hd))}
    bs = {n: torch.randn(ws[n].shape[0], generator=g) * 0.2 for n in "qkv"}
    wo = torch.randn(W, nh * hd, generator=g) * 0.2
    attn.qkv_weight = torch.cat([ws["q"], ws["k"], ws["v"]]).to(dtype).to(DEV)
    attn.qkv_bias = torch.cat([bs["q"], bs["k"], bs["v"]]).to(DEV)
    attn.o_weight = wo.to(dtype).to(DEV)
    pages = torch.zeros(2, 8, nkv, ps, hd, dtype=dtype, device=DEV)
    table = torch.tensor([[5, 2, 7, 0]], dtype=torch.int32, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    slots = (table[0].long()[pos.long() // ps] * ps + pos.long() % ps).to(torch.int32)
    zero = torch.zeros(T, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    batch = Batch(T, 1, zero, pos, zero, zero[:1], cu, zero[:0], 0, {0: GroupBatch(slots, table)}, [T], [T],
                  num_prefill_segs=1, max_prefill_q=T)
    got = attn.forward(h.to(DEV), batch, CacheView(group=0, k=pages[0], v=pages[1], page_size=ps)).cpu().float()
    pw = {f"{n}_proj.weight": ws[n].to(dtype).float() for n in "qkv"}
    pw.update({f"{n}_proj.bias": bs[n] for n in "qkv"})
    pw["o_proj.weight"] = wo.to(dtype).float()
    pcfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, rope_theta=777.0)
    want = plain.attention_block(h.float(), pw, "", torch.arange(T), pcfg, 5)
    assert torch.allclose(got, want, **t)


# ------------------------------------------------------------------ a toy mixer with state of its own
def test_a_toy_mixer_with_state_can_be_registered_built_and_stepped():
    """A mixer defined here - a decaying running mean of its inputs, kept per request in a
    fixed-size state slot - is registered, put into a model next to attention layers and stepped
    in portions and mixed batches, without any change to the package."""
    from pico_vllm_b200.parts import (Part, Param, Piece, FixedState, register, make, PreNormBlock, RMSNorm,
                                      GatedMLP, GQAAttention, Rotary, TokenEmbedding, OutputHead)
    from pico_vllm_b200.models import DecoderModel, LayerCall, Binding
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine import ModelRunner, StepItem, make_cache
    from pico_vllm_b200.weights import load_state_dict

    @register("mixer", "toy_running_mean")
    class RunningMean(Part):
        def __init__(self, width, decay):
            self.width, self.decay = width, decay
            self.mix = None

        def params(self):
            return [Param("mix", (Piece("mix", (self.width, self.width)),))]

        def cache_spec(self):
            return FixedState((self.width,), "float32")

        def forward(self, h, batch, cache):
            out = torch.empty_like(h)
            at = 0
            slots = batch.seg_slots.tolist()
            for s, n in enumerate(batch.q_lens):           # tokens of a segment in order
                state = cache.state[slots[s]]
                for i in range(at, at + n):
                    state.mul_(self.decay).add_(h[i].float() * (1 - self.decay))
                    out[i] = state.to(h.dtype)
                at += n
            return out @ self.mix.t()

    W, V = 32, 50
    embed = TokenEmbedding(V, W)
    toy = make("mixer", "toy_running_mean", width=W, decay=0.75)
    attn = GQAAttention(W, 2, 1, 16, position=Rotary(16, 100.0))
    blocks = [PreNormBlock(RMSNorm(W, 1e-5), toy, RMSNorm(W, 1e-5), GatedMLP(W, 48)),
              PreNormBlock(RMSNorm(W, 1e-5), attn, RMSNorm(W, 1e-5), GatedMLP(W, 48))]
    names = []
    bindings = [Binding(embed, {"weight": "emb"})]
    for i, b in enumerate(blocks):
        for pn, part in b.parts().items():
            bindings.append(Binding(part, {pc.key: f"l{i}.{pn}.{pc.key}" for p in part.params() for pc in p.pieces}))
    fn = RMSNorm(W, 1e-5)
    bindings.append(Binding(fn, {"weight": "fn"}))
    head = OutputHead(V, W, tied_to=embed)
    # the order names the attention block twice: its second call has a cache entry of its own
    order = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(1, 2)]

    class Cfg:
        architecture = "ToyForTest"
        max_position_embeddings = 256
    model = DecoderModel(Cfg(), embed, blocks, order, fn, head, bindings)
    g = torch.Generator().manual_seed(3)
    tensors = {}
    for b in bindings:
        for p in b.part.params():
            for pc in p.pieces:
                t = torch.randn(pc.shape, generator=g) * 0.3
                tensors[b.names[pc.key]] = t + 1 if p.init == "one_plus_normal" else t
    ecfg = EngineConfig(dtype="float32", page_size=4, max_cache_tokens=256, max_num_seqs=3, use_cuda_graph=False,
                        device=DEV)
    load_state_dict(model, tensors, torch.float32, DEV)
    model.materialize(DEV, torch.float32)
    runner = ModelRunner(model, make_cache(model, ecfg), ecfg)
    ids = {"p": helpers.random_ids(23, V, 1), "q": helpers.random_ids(14, V, 2)}
    whole = helpers.replay(runner, helpers.trace_whole(ids))
    ref = {"p": whole[0], "q": whole[1]}
    steps = helpers.trace_mixed(ids, max_live=2, seed=4, chunk_sizes=(3, 2, 5))
    want = helpers.expected_logits(steps, ids, ref)
    for i, (gg, w) in enumerate(zip(helpers.replay(runner, steps), want)):
        helpers.assert_close_logits(gg, w, 5e-5, f"toy step {i}")
    # the state really matters: another decay gives other logits
    toy.decay = 0.5
    other = helpers.replay(runner, helpers.trace_whole({"p": ids["p"]}))[0]
    assert float((other - ref["p"]).abs().max()) > 1e-3


# ------------------------------------------- a toy feed-forward with routing, a toy position encoding
def test_a_toy_routed_feed_forward_and_a_toy_position_encoding():
    """Two more parts defined here and registered without a change to the package: a feed-forward
    that routes each token to one of three small gated experts (router logits in float32), and a
    rotary encoding whose angles run at a third of the speed.  A model of two blocks - attention
    with the slow rotation + the experts; windowed attention + the ordinary feed-forward - is
    stepped whole and in mixed portions and compared with the same model written out here with
    the plain functions."""
    from pico_vllm_b200.parts import (Part, Param, Piece, register, make, PreNormBlock, RMSNorm, GatedMLP,
                                      GQAAttention, Rotary, TokenEmbedding, OutputHead)
    from pico_vllm_b200.models import DecoderModel, LayerCall, Binding
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine import ModelRunner, make_cache
    from pico_vllm_b200.weights import load_state_dict

    @register("feed_forward", "toy_top1_experts")
    class Top1Experts(Part):
        def __init__(self, width, inner, experts):
            self.width, self.inner, self.experts = width, inner, experts
            self.router = self.gate_up = self.down = None

        def params(self):
            E, I, W = self.experts, self.inner, self.width
            return [Param("router", (Piece("router", (E, W)),)),
                    Param("gate_up", tuple(Piece(f"e{e}.{n}", (I, W)) for e in range(E) for n in ("gate", "up"))),
                    Param("down", tuple(Piece(f"e{e}.down", (W, I)) for e in range(E)))]

        def forward(self, h, batch):
            I, W = self.inner, self.width
            choice = (h.float() @ self.router.float().t()).argmax(-1)
            out = torch.zeros_like(h)
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    x = h[rows].float()
                    g = x @ self.gate_up[2 * e * I:(2 * e + 1) * I].float().t()
                    u = x @ self.gate_up[(2 * e + 1) * I:(2 * e + 2) * I].float().t()
                    out[rows] = ((g * torch.sigmoid(g) * u) @ self.down[e * W:(e + 1) * W].float().t()).to(h.dtype)
            return out

    @register("position", "toy_slow_rotary")
    class SlowRotary(Rotary):
        def __init__(self, head_dim, theta, slowdown):
            super().__init__(head_dim, theta)
            self.slowdown = slowdown

        def frequencies(self):
            return super().frequencies() / self.slowdown

    W, V, I, E, hd = 48, 61, 40, 3, 16
    embed = TokenEmbedding(V, W)
    experts = make("feed_forward", "toy_top1_experts", width=W, inner=24, experts=E)
    slow = make("position", "toy_slow_rotary", head_dim=hd, theta=300.0, slowdown=3.0)
    blocks = [PreNormBlock(RMSNorm(W, 1e-5), GQAAttention(W, 3, 1, hd, position=slow), RMSNorm(W, 1e-5), experts),
              PreNormBlock(RMSNorm(W, 1e-6), GQAAttention(W, 2, 2, hd, position=Rotary(hd, 5000.0), window=9),
                           RMSNorm(W, 1e-6), GatedMLP(W, I))]
    bindings = [Binding(embed, {"weight": "emb"})]
    for i, b in enumerate(blocks):
        for pn, part in b.parts().items():
            bindings.append(Binding(part, {pc.key: f"l{i}.{pn}.{pc.key}" for p in part.params() for pc in p.pieces}))
    fn = RMSNorm(W, 1e-5)
    bindings.append(Binding(fn, {"weight": "fn"}))
    head = OutputHead(V, W, tied_to=embed)

    class Cfg:
        architecture = "ToyRoutedForTest"
        max_position_embeddings = 256
    model = DecoderModel(Cfg(), embed, blocks, [LayerCall(0, 0), LayerCall(1, 1)], fn, head, bindings)
    g = torch.Generator().manual_seed(11)
    tensors = {}
    for b in bindings:
        for p in b.part.params():
            for pc in p.pieces:
                t = torch.randn(pc.shape, generator=g) * 0.3
                tensors[b.names[pc.key]] = t + 1 if p.init == "one_plus_normal" else t
    ecfg = EngineConfig(dtype="float32", page_size=4, max_cache_tokens=256, max_num_seqs=3, use_cuda_graph=False,
                        device=DEV)
    load_state_dict(model, tensors, torch.float32, DEV)
    model.materialize(DEV, torch.float32)
    runner = ModelRunner(model, make_cache(model, ecfg), ecfg)

    def attention(h, l, nh, nkv, theta, slowdown, window):
        T = h.shape[0]
        w = {k[len(f"l{l}.mixer."):]: v for k, v in tensors.items() if k.startswith(f"l{l}.mixer.")}
        q = (h @ w["q.weight"].T + w["q.bias"]).view(T, nh, hd)
        k = (h @ w["k.weight"].T + w["k.bias"]).view(T, nkv, hd)
        v = (h @ w["v.weight"].T + w["v.bias"]).view(T, nkv, hd)
        pos = torch.arange(T)
        cos, sin = plain.rotary_angles(pos.float() / slowdown, hd, theta)
        o = plain.attention_scores_softmax_pv(plain.apply_rotary(q, cos, sin), plain.apply_rotary(k, cos, sin), v, pos,
                                              window)
        return o.reshape(T, nh * hd) @ w["o.weight"].T

    routed = []

    def reference(ids):
        x = plain.embed(torch.tensor(ids), tensors["emb"])
        x = x + attention(plain.rms_norm(x, tensors["l0.norm1.weight"], 1e-5), 0, 3, 1, 300.0, 3.0, None)
        h = plain.rms_norm(x, tensors["l0.norm2.weight"], 1e-5)
        choice = (h @ tensors["l0.feed_forward.router"].T).argmax(-1)
        routed.append(choice)
        y = torch.zeros_like(h)
        for t in range(h.shape[0]):
            e = int(choice[t])
            w = {f"{n}_proj.weight": tensors[f"l0.feed_forward.e{e}.{n}"] for n in ("gate", "up", "down")}
            y[t] = plain.swiglu_mlp(h[t:t + 1], w, "")[0]
        x = x + y
        x = x + attention(plain.rms_norm(x, tensors["l1.norm1.weight"], 1e-6), 1, 2, 2, 5000.0, 1.0, 9)
        w = {f"{n}_proj.weight": tensors[f"l1.feed_forward.{n}.weight"] for n in ("gate", "up", "down")}
        x = x + plain.swiglu_mlp(plain.rms_norm(x, tensors["l1.norm2.weight"], 1e-6), w, "")
        return plain.rms_norm(x, tensors["fn"], 1e-5) @ tensors["emb"].T

    ids = {"p": helpers.random_ids(31, V, 7), "q": helpers.random_ids(18, V, 8), "r": helpers.random_ids(9, V, 9)}
    ref = {rid: reference(t) for rid, t in ids.items()}
    assert len(set(torch.cat(routed).tolist())) == E, "the test should reach every expert"
    for steps in (helpers.trace_whole(ids), helpers.trace_mixed(ids, max_live=3, seed=5, chunk_sizes=(4, 2, 7))):
        want = helpers.expected_logits(steps, ids, ref)
        for i, (gg, w) in enumerate(zip(helpers.replay(runner, steps), want)):
            if w is not None:
                helpers.assert_close_logits(gg, w, 5e-5, f"toy routed step {i}")
    assert all(gr.pool.in_use == 0 for gr in runner.cache.groups)


# ------------------------------------------------------------------ full portions of a prompt from a graph
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["b", "d"])
def test_full_portions_are_replayed_from_a_graph(dtype, name):
    """A step that is one portion of one prompt with the configured number of tokens is recorded once
    and replayed: here portions of 24 tokens of three requests, at changing places of their prompts, with
    no row, the last row or another row wanted, between steps of other shapes and with pages that come
    back from ended requests.  Portions that come after 40 tokens or more also get two blocks per query tile in
    the tensor-core attention kernel (configuration d in bfloat16), recorded and launched directly."""
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine import ModelRunner, make_cache, model_from_tensors
    cfg = helpers.tiny_config(name)
    P = 24
    ecfg = EngineConfig(dtype=dtype, page_size=helpers.TINY[name]["page_size"], max_cache_tokens=224, max_num_seqs=2,
                        use_cuda_graph=True, graph_prefill_tokens=P, pair_min_context=40, device=DEV)
    tensors = helpers.tiny_tensors(name, torch.float32 if dtype == "float32" else torch.bfloat16)
    model = model_from_tensors(cfg, tensors, ecfg)
    runner = ModelRunner(model, make_cache(model, ecfg, poison_freed=True), ecfg)
    reqs = {"x": helpers.random_ids(3 * P + 5, cfg.vocab_size, 41), "y": helpers.random_ids(2 * P, cfg.vocab_size, 42),
            "z": helpers.random_ids(P + 30 + 47, cfg.vocab_size, 43)}
    x, y, z = reqs["x"], reqs["y"], reqs["z"]
    steps = [dict(entries=[dict(id="x", tokens=x[:P], want=[])], end=[]),                       # recorded, no row
             dict(entries=[dict(id="y", tokens=y[:P], want=[P - 1])], end=[]),                   # recorded, one row
             dict(entries=[dict(id="x", tokens=x[P:2 * P], want=[7])], end=[]),                  # replayed, another row
             dict(entries=[dict(id="x", tokens=x[2 * P:3 * P], want=[])], end=[]),               # replayed
             dict(entries=[dict(id="x", tokens=x[3 * P:], want=[4]), dict(id="y", tokens=y[P:P + 3], want=[2])], end=["x"]),
             dict(entries=[dict(id="z", tokens=z[:30], want=[29])], end=[]),                     # other shape, x's pages
             dict(entries=[dict(id="z", tokens=z[30:30 + P], want=[P - 1])], end=[]),            # replayed, late place
             dict(entries=[dict(id="z", tokens=z[30 + P:], want=[0, 46])], end=["z"]),           # after 54 tokens, launched directly
             dict(entries=[dict(id="y", tokens=y[P + 3:], want=[P - 4])], end=["y"])]
    want = helpers.expected_logits(steps, reqs, _plain_logits(name, reqs, tensors))
    got = helpers.replay(runner, steps)
    for i, (g, w) in enumerate(zip(got, want)):
        assert (g is None) == (w is None), f"step {i}"
        if w is not None:
            helpers.assert_close_logits(g, w, REL[dtype], f"{name}/{dtype} step {i}")
    assert runner.graph_replays == 5
    assert all(g.pool.in_use == 0 for g in runner.cache.groups)
