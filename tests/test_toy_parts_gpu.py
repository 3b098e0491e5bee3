"""Toy parts defined here and stepped without a change to the package: what the interfaces for
another mixer, cache need, position encoding and launch plan have to carry.

* a mixer with per-request state, written with device-side torch operations only, stepped with
  graph replay on (decode buckets and full portions of a prompt): a recorded step runs its work
  once, so the state advances once;
* a mixer that keeps ONE latent vector per token in pages (a cache need of its own:
  ``PagedTensors``; no keys/values pair) and asks for scratch through ``plan``;
* a learned absolute position encoding added at the embedding stage;
* a rotary encoding that names a pairing the kernels do not have: refused, not computed wrongly;
* a norm of another kind (mean and variance, with a bias) and another arrangement of a layer
  (the norm AFTER each residual add), both defined here, around the package's attention and
  feed-forward.

None of these is a model of the reference or of anyone's; the reference has one mixer, one cache
shape and one position encoding (pico_vllm/model.py:126-227, pico_vllm/blockmanager.py:39-42).
"""
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _assemble(blocks, order, V, W, embed_position=None, seed=3, final_norm=None, dtype=torch.float32, scale=0.3):
    """A DecoderModel of the given blocks with random float32 tensors; returns (model, tensors)."""
    from pico_vllm_b200.parts import RMSNorm, TokenEmbedding, OutputHead
    from pico_vllm_b200.models import DecoderModel, Binding
    from pico_vllm_b200.weights import load_state_dict
    embed = TokenEmbedding(V, W)
    bindings = [Binding(embed, {"weight": "emb"})]
    if embed_position is not None:
        bindings.append(Binding(embed_position, {pc.key: f"pos.{pc.key}" for p in embed_position.params() for pc in p.pieces}))
    for i, b in enumerate(blocks):
        for pn, part in b.parts().items():
            bindings.append(Binding(part, {pc.key: f"l{i}.{pn}.{pc.key}" for p in part.params() for pc in p.pieces}))
    fn = final_norm if final_norm is not None else RMSNorm(W, 1e-5)
    bindings.append(Binding(fn, {pc.key: ("fn" if pc.key == "weight" else f"fn.{pc.key}") for p in fn.params() for pc in p.pieces}))
    head = OutputHead(V, W, tied_to=embed)

    class Cfg:
        architecture = "ToyForTest"
        max_position_embeddings = 256
    model = DecoderModel(Cfg(), embed, blocks, order, fn, head, bindings, embed_position=embed_position)
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for b in bindings:
        for p in b.part.params():
            for pc in p.pieces:
                t = torch.randn(pc.shape, generator=g) * scale
                tensors[b.names[pc.key]] = t + 1 if p.init == "one_plus_normal" else t
    if dtype != torch.float32:      # what a folder stored in 16 bits holds: the matrices rounded, the vectors as they are
        tensors = {k: (v.to(dtype).float() if v.dim() > 1 else v) for k, v in tensors.items()}
    load_state_dict(model, {k: (v.to(dtype) if v.dim() > 1 else v) for k, v in tensors.items()}, dtype, DEV)
    model.materialize(DEV, dtype)
    return model, tensors


def _runner(model, **options):
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine import ModelRunner, make_cache
    opts = dict(dtype="float32", page_size=4, max_cache_tokens=256, max_num_seqs=3, use_cuda_graph=False, device=DEV)
    opts.update(options)
    ecfg = EngineConfig(**opts)
    return ModelRunner(model, make_cache(model, ecfg, poison_freed=True), ecfg)


def _same_as_whole(model, ids, steps, **graph_options):
    """The given cutting (with ``graph_options``) against each request whole without graphs."""
    whole = helpers.replay(_runner(model), helpers.trace_whole(ids))
    ref = dict(zip(ids, whole))
    runner = _runner(model, **graph_options)
    want = helpers.expected_logits(steps, ids, ref)
    for i, (g, w) in enumerate(zip(helpers.replay(runner, steps), want)):
        assert (g is None) == (w is None)
        if w is not None:
            helpers.assert_close_logits(g, w, 5e-5, f"toy step {i}")
    return runner


# ------------------------------------------------------------------ state of its own, with graph replay
def test_a_toy_mixer_with_state_is_stepped_once_by_recorded_steps():
    from pico_vllm_b200.parts import (Part, Param, Piece, FixedState, register, make, PreNormBlock, RMSNorm, GatedMLP,
                                      GQAAttention, Rotary)
    from pico_vllm_b200.models import LayerCall

    @register("mixer", "toy_running_mean_on_device")
    class RunningMean(Part):
        """state = decay * state + (1 - decay) * h for every token in order; output = state @ mix^T.  Device-side
        operations only (no host reads), so a step can be recorded; rows with position -1 are padding."""

        def __init__(self, width, decay):
            self.width, self.decay = width, decay
            self.mix = None

        def params(self):
            return [Param("mix", (Piece("mix", (self.width, self.width)),))]

        def cache_spec(self):
            return FixedState((self.width,), "float32")

        def forward(self, h, batch, cache):
            st, d = cache.state, self.decay
            slots = batch.seg_slots.long()
            if batch.decode_only:                      # one token per segment, maybe padded: all rows at once
                valid = (batch.positions >= 0).unsqueeze(1)
                old = st.index_select(0, slots)
                new = old * d + h.float() * (1 - d)
                st.index_add_(0, slots, torch.where(valid, new - old, torch.zeros_like(new)))
                out = torch.where(valid, new, torch.zeros_like(new))
            else:
                out = torch.empty(h.shape, dtype=torch.float32, device=h.device)
                at = 0
                for s, n in enumerate(batch.q_lens):   # the host knows the segments' lengths
                    slot = slots[s:s + 1]
                    state = st.index_select(0, slot)
                    for i in range(at, at + n):
                        state = state * d + h[i:i + 1].float() * (1 - d)
                        out[i:i + 1] = state
                    st.index_copy_(0, slot, state)
                    at += n
            return out.to(h.dtype) @ self.mix.t()

    W, V, P = 32, 50, 8
    toy = make("mixer", "toy_running_mean_on_device", width=W, decay=0.75)
    attn = GQAAttention(W, 2, 1, 16, position=Rotary(16, 100.0))
    blocks = [PreNormBlock(RMSNorm(W, 1e-5), toy, RMSNorm(W, 1e-5), GatedMLP(W, 48)),
              PreNormBlock(RMSNorm(W, 1e-5), attn, RMSNorm(W, 1e-5), GatedMLP(W, 48))]
    model, _ = _assemble(blocks, [LayerCall(0, 0), LayerCall(1, 1)], V, W)
    ids = {"p": helpers.random_ids(3 * P + 9, V, 1), "q": helpers.random_ids(P + 6, V, 2),
           "r": helpers.random_ids(11, V, 3)}
    p, q, r = ids["p"], ids["q"], ids["r"]
    one = lambda rid, toks, end=False: dict(entries=[dict(id=rid, tokens=toks, want=[len(toks) - 1])],
                                            end=[rid] if end else [])
    steps = [one("p", p[:P]), one("q", q[:P]), one("p", p[P:2 * P]), one("p", p[2 * P:3 * P]),   # full portions: recorded, replayed
             one("r", r[:10])]
    # then single tokens: one, two and three requests at a time (buckets 1, 2 and 4; the first step of each records)
    for i in range(6):
        entries = [dict(id="p", tokens=[p[3 * P + i]], want=[0])]
        if i >= 1:
            entries.append(dict(id="q", tokens=[q[P + i - 1]], want=[0]))
        if i == 5:
            entries.append(dict(id="r", tokens=[r[10]], want=[0]))
        steps.append(dict(entries=entries, end=["r"] if i == 5 else []))
    for i in range(6, 9):
        steps.append(dict(entries=[dict(id="p", tokens=[p[3 * P + i]], want=[0])], end=["p"] if i == 8 else []))
    steps.append(one("q", q[P + 5:], end=True))
    runner = _same_as_whole(model, ids, steps, use_cuda_graph=True, graph_prefill_tokens=P, max_num_batched_tokens=64)
    assert runner.graph_replays >= 12
    assert len(runner._graphs) >= 4           # portions with one wanted row, buckets 1, 2 and 4


# ------------------------------------------------------------------ a cache need and scratch of its own
def test_a_toy_mixer_with_pages_of_its_own_shape_and_scratch_of_its_own():
    """One latent vector per token in pages (no keys/values pair), read back through the block table; its
    plan asks the step function for scratch, which arrives as ``batch.scratch``.  Nothing under ``engine/`` or
    ``cache/`` knows this mixer."""
    from pico_vllm_b200.parts import (Part, Param, Piece, PagedTensors, MixerPlan, register, make, PreNormBlock,
                                      RMSNorm, GatedMLP, GQAAttention, Rotary)
    from pico_vllm_b200.models import LayerCall
    asked = []

    @register("mixer", "toy_latent_mean")
    class LatentMean(Part):
        """latent_t = h_t @ down^T is stored per token; output_t = mean of the latents 0..t, through ``up``."""

        def __init__(self, width, latent):
            self.width, self.latent = width, latent
            self.down = self.up = None

        def params(self):
            return [Param("down", (Piece("down", (self.latent, self.width)),)),
                    Param("up", (Piece("up", (self.width, self.latent)),))]

        def cache_spec(self):
            return PagedTensors((("latent", (self.latent,)),))

        def plan(self, shape):
            need = shape.num_tokens * self.latent
            asked.append(need)
            return MixerPlan(key=(), scratch_floats=need)

        def forward(self, h, batch, cache):
            T = h.shape[0]
            gb = batch.groups[cache.group]
            pages = cache.tensors["latent"]                    # [num_pages, page_size, latent]
            flat = pages.view(-1, self.latent)
            lat = h.float() @ self.down.float().t()
            flat.index_copy_(0, gb.slots.long(), lat.to(flat.dtype))
            assert batch.plan(self) is not None and batch.scratch is not None and batch.scratch.numel() >= T * self.latent
            acc = batch.scratch[:T * self.latent].view(T, self.latent)      # the scratch this mixer planned for
            ps = cache.page_size
            pos, seg = batch.positions.tolist(), batch.tok_seg.tolist()
            for t in range(T):
                n = torch.arange(pos[t] + 1, device=h.device)
                rows = gb.block_table[seg[t]].long()[n // ps] * ps + n % ps
                acc[t] = flat.index_select(0, rows).float().mean(0)
            return (acc @ self.up.float().t()).to(h.dtype)

    W, V = 32, 40
    toy = make("mixer", "toy_latent_mean", width=W, latent=12)
    attn = GQAAttention(W, 2, 2, 16, position=Rotary(16, 500.0))
    blocks = [PreNormBlock(RMSNorm(W, 1e-5), toy, RMSNorm(W, 1e-5), GatedMLP(W, 48)),
              PreNormBlock(RMSNorm(W, 1e-5), attn, RMSNorm(W, 1e-5), GatedMLP(W, 48))]
    model, _ = _assemble(blocks, [LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2)], V, W, seed=5)
    ids = {"p": helpers.random_ids(27, V, 1), "q": helpers.random_ids(14, V, 2), "r": helpers.random_ids(9, V, 3)}
    steps = helpers.trace_mixed(ids, max_live=3, seed=4, chunk_sizes=(3, 2, 5, 8))
    runner = _same_as_whole(model, ids, steps, max_cache_tokens=helpers.live_token_peak(steps, 4))
    # two groups of pages: the latents (two entries of one shape) and the attention's keys and values
    shapes = sorted(tuple(sorted((n, tuple(t.shape[2:])) for n, t in g.tensors.items())) for g in runner.cache.groups)
    assert shapes == [(("k", (2, 4, 16)), ("v", (2, 4, 16))), (("latent", (4, 12)),)]
    assert [len(g.entries) for g in runner.cache.groups if "latent" in g.tensors] == [2]
    assert asked and all(g.pool.in_use == 0 for g in runner.cache.groups)


# ------------------------------------------------------------------ positions at the embedding stage
def test_a_toy_learned_position_encoding_at_the_embedding_stage():
    from pico_vllm_b200.parts import Part, Param, Piece, register, make, PreNormBlock, RMSNorm, GatedMLP, GQAAttention, NoPosition
    from pico_vllm_b200.models import LayerCall
    import plain_qwen2 as plain

    @register("position", "toy_learned_absolute")
    class LearnedAbsolute(Part):
        def __init__(self, width, max_positions):
            self.width, self.max_positions = width, max_positions
            self.table = None

        def params(self):
            return [Param("table", (Piece("table", (self.max_positions, self.width)),))]

        def add_to(self, x, positions):
            return x + self.table.float().index_select(0, positions.clamp(min=0).long())

    W, V, hd = 32, 45, 16
    pos = make("position", "toy_learned_absolute", width=W, max_positions=64)
    blocks = [PreNormBlock(RMSNorm(W, 1e-5), GQAAttention(W, 2, 1, hd, position=NoPosition(hd)), RMSNorm(W, 1e-5),
                           GatedMLP(W, 40))]
    model, tensors = _assemble(blocks, [LayerCall(0, 0)], V, W, embed_position=pos, seed=9)

    def reference(ids):
        T = len(ids)
        x = plain.embed(torch.tensor(ids), tensors["emb"]) + tensors["pos.table"][:T]
        h = plain.rms_norm(x, tensors["l0.norm1.weight"], 1e-5)
        w = {k[len("l0.mixer."):]: v for k, v in tensors.items() if k.startswith("l0.mixer.")}
        q = (h @ w["q.weight"].T + w["q.bias"]).view(T, 2, hd)
        k = (h @ w["k.weight"].T + w["k.bias"]).view(T, 1, hd)
        v = (h @ w["v.weight"].T + w["v.bias"]).view(T, 1, hd)
        o = plain.attention_scores_softmax_pv(q, k, v, torch.arange(T))           # no rotation: positions came earlier
        x = x + o.reshape(T, 2 * hd) @ w["o.weight"].T
        mw = {f"{n}_proj.weight": tensors[f"l0.feed_forward.{n}.weight"] for n in ("gate", "up", "down")}
        x = x + plain.swiglu_mlp(plain.rms_norm(x, tensors["l0.norm2.weight"], 1e-5), mw, "")
        return plain.rms_norm(x, tensors["fn"], 1e-5) @ tensors["emb"].T

    ids = {"p": helpers.random_ids(29, V, 1), "q": helpers.random_ids(12, V, 2)}
    ref = {rid: reference(t) for rid, t in ids.items()}
    runner = _runner(model, use_cuda_graph=True)
    for steps in (helpers.trace_whole(ids), helpers.trace_mixed(ids, max_live=2, seed=2, chunk_sizes=(4, 2, 7))):
        want = helpers.expected_logits(steps, ids, ref)
        for i, (g, w) in enumerate(zip(helpers.replay(runner, steps), want)):
            helpers.assert_close_logits(g, w, 5e-5, f"learned positions step {i}")
    # the table matters: without it the same model gives other logits
    tensors["pos.table"] = torch.zeros_like(tensors["pos.table"])
    assert float((reference(ids["p"]) - ref["p"]).abs().max()) > 1e-3


# ------------------------------------------------------------------ a pairing the kernels do not have
def test_a_rotary_pairing_the_kernels_lack_is_refused():
    from pico_vllm_b200 import ops
    from pico_vllm_b200.errors import KernelError
    from pico_vllm_b200.engine import StepItem
    from pico_vllm_b200.parts import PreNormBlock, RMSNorm, GatedMLP, GQAAttention, Rotary
    from pico_vllm_b200.models import LayerCall
    W, V = 32, 30
    blocks = [PreNormBlock(RMSNorm(W, 1e-5), GQAAttention(W, 2, 1, 16, position=Rotary(16, 100.0, pairing="interleaved")),
                           RMSNorm(W, 1e-5), GatedMLP(W, 48))]
    model, _ = _assemble(blocks, [LayerCall(0, 0)], V, W)
    runner = _runner(model)
    slot = runner.cache.acquire("x")
    for toks in ([1, 2, 3, 4, 5], [7]):
        with pytest.raises(KernelError, match="pairing"):
            runner.step([StepItem(slot, toks, (0,))])
    runner.cache.check()
    # the fused small-batch kernel of the bfloat16 path refuses it too
    x = torch.zeros(2, 32, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(64, 32, dtype=torch.bfloat16, device=DEV)
    pos = torch.zeros(2, dtype=torch.int32, device=DEV)
    inv = torch.zeros(8, dtype=torch.float32, device=DEV)
    with pytest.raises(KernelError, match="pairing"):
        ops.skinny_qkv_rope_store(x, w, None, pos, inv, None, None, None, 2, 1, 16, 4, pairing="interleaved")


# ------------------------------------------------------------------ another norm, another arrangement
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_norm_with_bias_in_a_post_norm_arrangement(dtype):
    """The norm kind and the arrangement of a layer are parts like the others: a norm with mean, variance and
    bias (``add_norm(x, delta, rows)`` is all a norm has to offer) and a block that norms AFTER each add
    (``parts()`` and ``forward(x, pending, batch, cache) -> (x, pending)`` are all a block has to offer), around
    the package's own attention and feed-forward, stepped whole, in mixed portions and from recorded graphs."""
    from pico_vllm_b200.parts import Part, Param, Piece, register, make, GatedMLP, GQAAttention, Rotary
    from pico_vllm_b200.models import LayerCall
    import plain_qwen2 as plain
    import torch.nn.functional as F

    @register("norm", "toy_layer_norm")
    class LayerNormWithBias(Part):
        def __init__(self, width, eps):
            self.width, self.eps = width, eps
            self.weight = self.bias = None
            self.act_dtype = torch.float32

        def params(self):
            return [Param("weight", (Piece("weight", (self.width,)),), kind="vector", init="one_plus_normal"),
                    Param("bias", (Piece("bias", (self.width,)),), kind="vector")]

        def materialize(self, device, dtype):
            self.act_dtype = dtype

        def stream(self, x, delta):
            """norm(x + delta) as the new float32 residual stream (what a post-norm arrangement asks of its norm)."""
            return F.layer_norm(x + delta.float(), (self.width,), self.weight.float(), self.bias.float(), self.eps)

        def add_norm(self, x, delta, rows=None):
            """What every norm offers: activations for the next part (here only the head asks)."""
            if rows is not None:
                r = rows.long()
                x = x[r] + (delta[r].float() if delta is not None else 0)
            elif delta is not None:
                x += delta.float()
            return F.layer_norm(x, (self.width,), self.weight.float(), self.bias.float(), self.eps).to(self.act_dtype)

    class PostNormBlock:
        def __init__(self, mixer, norm1, feed_forward, norm2):
            self.mixer, self.norm1, self.feed_forward, self.norm2 = mixer, norm1, feed_forward, norm2

        def parts(self):
            return {"mixer": self.mixer, "norm1": self.norm1, "feed_forward": self.feed_forward, "norm2": self.norm2}

        def forward(self, x, pending, batch, cache):
            assert pending is None
            x = self.norm1.stream(x, self.mixer.forward(x.to(self.norm1.act_dtype), batch, cache))
            x = self.norm2.stream(x, self.feed_forward.forward(x.to(self.norm2.act_dtype), batch))
            return x, None

    W, V, hd, I = 48, 64, 16, 40         # sizes the small-batch kernels take: a norm they cannot compute must not reach them
    tdtype, tolerance = (torch.float32, 5e-5) if dtype == "float32" else (torch.bfloat16, 3e-2)
    def norm(eps):
        return make("norm", "toy_layer_norm", width=W, eps=eps)
    blocks = [PostNormBlock(GQAAttention(W, 2, 1, hd, position=Rotary(hd, 700.0)), norm(1e-5), GatedMLP(W, I), norm(1e-4)),
              PostNormBlock(GQAAttention(W, 4, 2, hd, position=Rotary(hd, 9000.0), window=11), norm(1e-6), GatedMLP(W, I),
                            norm(1e-5))]
    # matrices of scale 0.12: the parts' outputs stay of the size of the normed stream they are added to (at 0.3 a
    # feed-forward output is 25 against a stream of 3, and its rounding to bfloat16 alone is 1 % of the stream)
    model, tensors = _assemble(blocks, [LayerCall(0, 0), LayerCall(1, 1)], V, W, seed=21, final_norm=norm(1e-5),
                               dtype=tdtype, scale=0.12)

    if dtype == "bfloat16":
        # the head would take an RMS norm of these sizes into its own kernel; the toy norm it leaves alone
        from pico_vllm_b200.parts import RMSNorm
        rms = RMSNorm(W, 1e-5)
        rms.weight = torch.ones(W, device=DEV)
        stream = torch.zeros(4, W, device=DEV)
        assert model.head.can_fuse_norm(stream, rms, 4) and not model.head.can_fuse_norm(stream, model.final_norm, 4)

    def ln(x, name, eps):
        return F.layer_norm(x, (W,), tensors[f"{name}.weight" if name != "fn" else "fn"], tensors[f"{name}.bias"], eps)

    def attention(h, l, nh, nkv, theta, window):
        T = h.shape[0]
        w = {k[len(f"l{l}.mixer."):]: v for k, v in tensors.items() if k.startswith(f"l{l}.mixer.")}
        q = (h @ w["q.weight"].T + w["q.bias"]).view(T, nh, hd)
        k = (h @ w["k.weight"].T + w["k.bias"]).view(T, nkv, hd)
        v = (h @ w["v.weight"].T + w["v.bias"]).view(T, nkv, hd)
        pos = torch.arange(T)
        cos, sin = plain.rotary_angles(pos.float(), hd, theta)
        o = plain.attention_scores_softmax_pv(plain.apply_rotary(q, cos, sin), plain.apply_rotary(k, cos, sin), v, pos, window)
        return o.reshape(T, nh * hd) @ w["o.weight"].T

    def reference(ids):
        x = plain.embed(torch.tensor(ids), tensors["emb"])
        for l, (nh, nkv, theta, window, e1, e2) in enumerate([(2, 1, 700.0, None, 1e-5, 1e-4), (4, 2, 9000.0, 11, 1e-6, 1e-5)]):
            x = ln(x + attention(x, l, nh, nkv, theta, window), f"l{l}.norm1", e1)
            mw = {f"{n}_proj.weight": tensors[f"l{l}.feed_forward.{n}.weight"] for n in ("gate", "up", "down")}
            x = ln(x + plain.swiglu_mlp(x, mw, ""), f"l{l}.norm2", e2)
        return ln(x, "fn", 1e-5) @ tensors["emb"].T

    ids = {"p": helpers.random_ids(33, V, 4), "q": helpers.random_ids(14, V, 5), "r": helpers.random_ids(21, V, 6)}
    ref = {rid: reference(t) for rid, t in ids.items()}
    for options in (dict(use_cuda_graph=False), dict(use_cuda_graph=True, graph_batch_sizes=(1, 2, 4), graph_prefill_tokens=7)):
        runner = _runner(model, dtype=dtype, **options)
        for steps in (helpers.trace_whole(ids), helpers.trace_tail_decode(ids, 6),
                      helpers.trace_mixed(ids, max_live=3, seed=8, chunk_sizes=(7, 2, 7, 3))):
            want = helpers.expected_logits(steps, ids, ref)
            for i, (g, w) in enumerate(zip(helpers.replay(runner, steps), want)):
                if w is not None:
                    helpers.assert_close_logits(g, w, tolerance, f"post-norm step {i}")
        assert all(gr.pool.in_use == 0 for gr in runner.cache.groups)
    # the bias matters: without it the same model gives other logits
    tensors["l0.norm1.bias"] = torch.zeros_like(tensors["l0.norm1.bias"])
    assert float((reference(ids["p"]) - ref["p"]).abs().max()) > 1e-3
