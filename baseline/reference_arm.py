"""The reference arm of bench.py: the unmodified Koas-W/Pico-vLLM engine, driven through its own
public calls on the same shape, dtype, batch, context, steps and warm-up as the other arm.

"Installing" the reference is copying its ``pico_vllm`` folder to ``baseline/_ref/``: the project
has no setup.py or pyproject.toml, and its own scripts import the modules by bare name from
inside that folder (pico_vllm/run_single.py:1-7).  This file puts that folder on ``sys.path`` and
follows pico_vllm/run_single.py:10-37 line by line: ``ModelConfig()`` -> ``Qwen25_15B`` ->
``load_weights(model, folder)`` -> ``.to(bfloat16).to("cuda")`` -> ``BlockManager`` ->
``Engine(..., use_cuda_graph=True)`` -> ``submit`` / ``step``.  The weights folder is a random
Qwen2.5-1.5B-shaped model written here with torch and safetensors alone (the same tensor names
the reference's loader reads, pico_vllm/weights.py:18-68); the tokenizer is a three-method
stand-in (``encode`` / ``decode`` / ``eos_token_id``: all the engine uses,
pico_vllm/engine.py:48,254,381).  Nothing of this repository's package is imported here.

Where a stock limit differs from the measured configuration the difference is named in the
printed ``config``: the scheduler admits 4 requests unless its public ``max_num_seqs`` attribute is
raised (pico_vllm/scheduler.py:84), the graph holds ``max_batch_size`` = 8 rows
(pico_vllm/engine.py:20), a request's cache holds 4096 tokens (pico_vllm/engine.py:41), prompts run
whole, one forward each (pico_vllm/engine.py:299-357), and the prefix cache is switched off
(``enable_prefix_cache=False``) because random prompts share nothing.
"""
import json
import os
import shutil
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref", "pico_vllm")

SHAPE = dict(vocab_size=151936, hidden_size=1536, num_hidden_layers=28, num_attention_heads=12,
             num_key_value_heads=2, intermediate_size=8960)


class StandInTokenizer:
    """Token ids in, token ids out: ``encode`` takes a list of ids (or digits separated by blanks),
    ``decode`` joins ids with blanks, and no id is the end token."""
    eos_token_id = -1

    def encode(self, prompt):
        if isinstance(prompt, str):
            return [int(t) for t in prompt.split()]
        return list(prompt)

    def decode(self, ids):
        return " ".join(str(int(t)) for t in ids)


def ensure_reference():
    """``baseline/_ref/pico_vllm`` must hold an unmodified copy of the reference's ``pico_vllm`` folder; when it
    does not and PICO_REFERENCE_SOURCE names a checkout of the reference, the folder is copied from there."""
    if os.path.isfile(os.path.join(REF_DIR, "engine.py")):
        return
    source = os.environ.get("PICO_REFERENCE_SOURCE")
    if source and os.path.isdir(os.path.join(source, "pico_vllm")):
        os.makedirs(os.path.dirname(REF_DIR), exist_ok=True)
        shutil.copytree(os.path.join(source, "pico_vllm"), REF_DIR)
        return
    raise FileNotFoundError("baseline/_ref/pico_vllm is missing: copy the reference's pico_vllm folder there "
                            "(or set PICO_REFERENCE_SOURCE to a checkout of the reference)")


def write_random_weights(folder, layers, seed=0):
    """model.safetensors with the tensor names of a Qwen2 model folder: N(0, 0.02), norm weights
    1 + N(0, 0.02), bfloat16."""
    import torch
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)
    H, I, V = SHAPE["hidden_size"], SHAPE["intermediate_size"], SHAPE["vocab_size"]
    hd = H // SHAPE["num_attention_heads"]
    q, kv = SHAPE["num_attention_heads"] * hd, SHAPE["num_key_value_heads"] * hd

    def n(*shape):
        return (torch.randn(*shape, generator=g) * 0.02).to(torch.bfloat16)

    def one(*shape):
        return (1.0 + torch.randn(*shape, generator=g) * 0.02).to(torch.bfloat16)

    w = {"model.embed_tokens.weight": n(V, H), "model.norm.weight": one(H)}
    for i in range(layers):
        p = f"model.layers.{i}."
        for name, rows in (("q", q), ("k", kv), ("v", kv)):
            w[f"{p}self_attn.{name}_proj.weight"] = n(rows, H)
            w[f"{p}self_attn.{name}_proj.bias"] = n(rows)
        w[p + "self_attn.o_proj.weight"] = n(H, q)
        w[p + "mlp.gate_proj.weight"] = n(I, H)
        w[p + "mlp.up_proj.weight"] = n(I, H)
        w[p + "mlp.down_proj.weight"] = n(H, I)
        w[p + "input_layernorm.weight"] = one(H)
        w[p + "post_attention_layernorm.weight"] = one(H)
    save_file(w, os.path.join(folder, "model.safetensors"))


def _scratch_dir(need_bytes):
    try:
        st = os.statvfs("/dev/shm")
        if st.f_bavail * st.f_frsize > need_bytes and os.access("/dev/shm", os.W_OK):
            return "/dev/shm"
    except OSError:
        pass
    return None


def _say(msg):
    print(f"[bench reference] {msg}", file=sys.stderr, flush=True)


def load_reference_model(layers):
    """pico_vllm/run_single.py:10-13 with a random weights folder."""
    import torch
    from model import Qwen25_15B, ModelConfig
    from weights import load_weights
    cfg = ModelConfig()
    if layers != cfg.num_hidden_layers:
        cfg.num_hidden_layers = layers
    tmp = tempfile.mkdtemp(prefix="pico_ref_", dir=_scratch_dir(4 << 30))
    try:
        t0 = time.time()
        write_random_weights(tmp, layers)
        _say(f"random {layers}-layer weights written in {time.time() - t0:.0f} s")
        t0 = time.time()
        model = Qwen25_15B(cfg)
        model = load_weights(model, tmp)
        model = model.to(torch.bfloat16).to("cuda")
        _say(f"reference model built and loaded in {time.time() - t0:.0f} s")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return cfg, model


def make_engine(cfg, model, batch, context):
    """pico_vllm/run_single.py:17-29 with as many pages as the batch needs; returns (engine, notes)."""
    import torch
    from blockmanager import BlockManager
    from cache import PagedKVCache
    from engine import Engine
    notes = []
    blocks = batch * (-(-(context + 16) // 16)) + 64
    bm = BlockManager(num_gpu_blocks=blocks, num_cpu_blocks=0, block_size=16, num_layers=cfg.num_hidden_layers,
                      num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, dtype=torch.bfloat16)
    kwargs = {}
    if batch > 8:
        kwargs["max_batch_size"] = batch        # a constructor argument; the stock default is 8
        notes.append(f"max_batch_size={batch} (stock 8)")
    if context > 4096:
        kwargs["cache_kwargs"] = dict(block_manager=bm, num_layers=cfg.num_hidden_layers, max_seq_len=context,
                                      num_kv_heads=cfg.local_num_key_value_heads, head_dim=cfg.head_dim,
                                      device="cuda", dtype=torch.bfloat16)
        notes.append(f"cache max_seq_len={context} (stock 4096)")
    engine = Engine(model=model, tokenizer=StandInTokenizer(), block_manager=bm, cache_cls=PagedKVCache,
                    device="cuda", use_cuda_graph=True, enable_prefix_cache=False, **kwargs)
    if batch > engine.scheduler.max_num_seqs:
        engine.scheduler.max_num_seqs = batch   # a public attribute; the stock value is 4
        notes.append(f"scheduler.max_num_seqs={batch} (stock 4)")
    return engine, bm, notes


def decode_run(cfg, model, batch, context, steps, warmup, seed):
    """``batch`` requests with prompts of context - steps - warmup - 1 tokens; after the prompts and
    the warm-up steps, ``steps`` calls of ``Engine.step`` are timed on the device (CUDA events) and
    on the host clock.  Returns (device ms per step, wall ms per step, notes)."""
    import torch
    engine, bm, notes = make_engine(cfg, model, batch, context)
    g = torch.Generator().manual_seed(seed)
    prompt_len = context - steps - warmup - 1
    for _ in range(batch):
        ids = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist()
        engine.submit(ids, max_new_tokens=steps + warmup + 64, temperature=0, top_p=1.0)
    while len(engine.scheduler.decoding) < batch or engine.scheduler.prefilling:
        engine.step()                       # prompts, whole, one forward each
        if not (engine.scheduler.waiting or engine.scheduler.prefilling or engine.scheduler.decoding):
            raise RuntimeError("the reference engine lost its requests before decoding")
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    t0.record()
    for _ in range(steps):
        done = engine.step()
        if done:
            raise RuntimeError("a request ended inside the timed region")
    t1.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - w0) * 1000.0 / steps
    dev = t0.elapsed_time(t1) / steps
    if len(engine.scheduler.decoding) != batch:
        raise RuntimeError("not every request was decoding in the timed region")
    del engine, bm
    torch.cuda.empty_cache()
    return dev, wall, notes


def prefill_run(cfg, model, T, reps, seed):
    """One prompt of T tokens through ``submit`` + ``step`` (the step that runs the prompt and samples
    its first token); median device time of ``reps`` runs after 3 warm-up runs."""
    import torch
    engine, bm, _ = make_engine(cfg, model, 1, max(T + 64, 256))
    g = torch.Generator().manual_seed(seed)
    times = []
    for i in range(reps + 3):
        ids = torch.randint(0, cfg.vocab_size, (T,), generator=g).tolist()
        engine.submit(ids, max_new_tokens=1, temperature=0, top_p=1.0)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        done = engine.step()
        t1.record()
        torch.cuda.synchronize()
        if len(done) != 1:
            raise RuntimeError("the prompt's step did not complete its request")
        # the finished request passes through the decoding list once more before it is closed and its pages
        # are given back (pico_vllm/scheduler.py:157-170)
        while engine.scheduler.prefilling or engine.scheduler.decoding:
            engine.step()
        if i >= 3:
            times.append(t0.elapsed_time(t1))
    del engine, bm
    torch.cuda.empty_cache()
    times.sort()
    return times[len(times) // 2]


def run(args, peaks, clock_sampler, prefill_flops, published_b1):
    """Prints the bench line of the reference arm (or its ``unavailable`` line) and returns 0."""
    try:
        ensure_reference()
        if REF_DIR not in sys.path:
            sys.path.insert(0, REF_DIR)
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        batch, context, layers = args.batch, args.context, args.layers
        with torch.no_grad():
            cfg, model = load_reference_model(layers)
            clock_sampler.start()
            ms, wall_ms, notes = decode_run(cfg, model, batch, context, args.steps, args.warmup, seed=1)
            clocks = clock_sampler.stop()
            _say(f"decode batch {batch}: {ms:.3f} ms per step on the device, {wall_ms:.3f} ms on the host clock")
            T = 2048
            pre_ms = prefill_run(cfg, model, T, reps=5, seed=3)
            _say(f"prefill {T}: {pre_ms:.2f} ms")
            points = {}
            if not args.no_points:
                for b in (1, 64):
                    pms, _, pn = decode_run(cfg, model, b, context, 32, 8, seed=10 + b)
                    points[f"decode_b{b}"] = round(b / pms * 1000.0, 1)
                    points[f"decode_b{b}_ms"] = round(pms, 4)
                    notes += [x for x in pn if x not in notes]
    except Exception as e:                                  # the attempt's own exception, in one line
        msg = " ".join(f"{type(e).__name__}: {e}".split())
        print(json.dumps({"impl": "reference", "unavailable": msg[:400]}))
        return 0
    wbytes = sum(p.numel() * p.element_size() for p in model.parameters())
    kvb = 2 * layers * cfg.num_key_value_heads * cfg.head_dim * 2
    step_bytes = wbytes + batch * (context - args.steps / 2) * kvb
    achieved = step_bytes / (ms / 1000.0) / 1e9
    flops = prefill_flops(T, layers)
    out = {
        "metric": f"decode tok/s (Qwen2.5-1.5B shape, batch {batch}, context {context})",
        "value": round(batch / ms * 1000.0, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)", "impl": "reference",
        "config": {"model": "Qwen2.5-1.5B shape", "layers": layers, "layers_full": 28,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied": cfg.tie_word_embeddings, "global_batch": batch, "seq_len": context, "page_size": 16,
                   "parallelism": "single GPU", "cuda_graph": True, "prefix_cache": False,
                   "l2": "no flush: each step reads >3 GB of weights and cache, L2 is 126 MB",
                   "peaks": peaks["source"],
                   "reference_limits": "; ".join(notes) if notes else "stock"},
        "clocks": clocks,
        # Engine.step takes host token ids (python lists) and returns after reading the sampled ids back
        # (.item() per row, pico_vllm/sampler.py:75-77): the same call is the device-timed and the end-to-end number
        "e2e": {"value": round(batch / wall_ms * 1000.0, 1), "unit": "tok/s", "ms_per_step": round(wall_ms, 4),
                "h2d_bytes_per_step": max(8, batch) * (8 + 4 + 8 + 4), "d2h_bytes_per_step": 8 * batch},
        "gpu_launches": None,
        "prefill": {"value": round(T / pre_ms * 1000.0, 1), "tokens": T, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms / 1000.0) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "decode_b1_vs_published_97": (round(points["decode_b1"] / published_b1, 2) if "decode_b1" in points else None),
    }
    print(json.dumps(out))
    return 0
