"""Benchmark of the serving step: decode tokens per second on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: the layer sizes of the Qwen2.5-1.5B shape (28 layers, width 1536, 12 query and 2
key/value heads of 128, feed-forward 8960, vocabulary 151936, tied head) with random weights,
bfloat16, a batch of 8 requests decoding at a context of 4096 tokens.  A "step" is one decode
step of the whole batch.  Prints ONE JSON line:

* ``value``: decoded tokens per second, timed on the device with CUDA events around K steps of
  the step function (batch building, index upload and graph replay included);
* ``e2e``: the same through the Python entry point (``LLM.submit`` / ``LLM.step``), host token
  ids in, sampled host token ids out, every step;
* ``prefill``: one 2,048-token prompt through the step function;
* ``roofline``: bytes a decode step has to read (every weight once, the cache of the live
  requests) / its time, against the measured copy bandwidth;
* ``points``: decode at batch 1 and 64 at the same context (tokens per second, ms per step, fraction of the
  roofline), and the reference's own decode workload - a 512-token prompt, then 256 generated tokens, the 256
  steps timed - at batch 1, 8 and 64 (``gen256_b*``).

Every timed decode step also chooses its tokens (greedy; for up to 16 rows inside the head's kernel).
``--config 3b`` and ``--config 7b`` run the two larger shapes of the architecture with the workloads named for
them (``run_shape``); ``--impl reference`` runs the unmodified reference engine (``baseline/reference_arm.py``).

The weights and the cache of every timed step are far larger than the 126 MB L2, so no L2 flush
is needed between iterations (``config.l2`` says so).  Peaks come from MEASURED_PEAKS.json when
the file is there, else from the fallback of an earlier measurement on this kind of GPU.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PROFILE_RANGE = None         # "decode" / "prefill": bracket that timed region with cudaProfilerStart/Stop
PUBLISHED_DECODE_B1 = 97.0   # tok/s, batch 1, the reference's README (other hardware)

MODEL = dict(architectures=["Qwen2ForCausalLM"], vocab_size=151936, hidden_size=1536, num_hidden_layers=28,
             num_attention_heads=12, num_key_value_heads=2, intermediate_size=8960, rope_theta=1000000.0,
             rms_norm_eps=1e-6, tie_word_embeddings=True, use_sliding_window=False,
             max_position_embeddings=32768, hidden_act="silu")
FULL_LAYERS = 28
# the two larger shapes of the same architecture (--config 3b / 7b): their own workloads, see run_shape
SHAPES = {
    "1.5b": ("Qwen2.5-1.5B shape", MODEL),
    "3b": ("Qwen2.5-3B shape", dict(MODEL, hidden_size=2048, num_hidden_layers=36, num_attention_heads=16,
                                    intermediate_size=11008)),
    "7b": ("Qwen2.5-7B shape", dict(MODEL, vocab_size=152064, hidden_size=3584, num_attention_heads=28,
                                    num_key_value_heads=4, intermediate_size=18944, tie_word_embeddings=False)),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")
    try:
        with open(path) as f:
            m = json.load(f)
        if "hbm_gbs" in m:
            out["hbm_gbs"] = float(m["hbm_gbs"])
        if "bf16_tflops" in m:
            out["bf16_tflops"] = float(m["bf16_tflops"])
        if "bf16_tflops_sustained" in m:
            out["bf16_tflops_sustained"] = float(m["bf16_tflops_sustained"])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """nvidia-smi in the background, sampling SM clock and throttle reasons every 200 ms."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                    power.append(float(parts[2]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.remove(self.path)
        except OSError:
            pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def scratch_dir(need_bytes):
    """A memory-backed folder when it has room (the model folder is written and read once)."""
    try:
        st = os.statvfs("/dev/shm")
        if st.f_bavail * st.f_frsize > need_bytes and os.access("/dev/shm", os.W_OK):
            return "/dev/shm"
    except OSError:
        pass
    return None


def make_model_folder(layers, folder):
    import torch
    from pico_vllm_b200.registry import config_from_dict
    from pico_vllm_b200.weights import write_random_model
    raw = dict(MODEL, num_hidden_layers=layers)
    cfg = config_from_dict(raw)
    t0 = time.time()
    write_random_model(cfg, seed=0, out_dir=folder, dtype="bfloat16")
    print(f"[bench] random {layers}-layer model written in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return cfg


def weight_bytes(model):
    """Bytes of every weight a decode step reads once (the embedding table counts once: it is
    the head's matrix when tied; the gather of a few rows is left out)."""
    seen, total = set(), 0
    for part in model.all_parts():
        for p in part.params():
            t = getattr(part, p.attr)
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
    return total


def kv_bytes_per_token(model, cache):
    return cache.bytes_per_page() // cache.page_size


def prefill_flops(cfg, T):
    H, I, V, L = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers
    nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    per_tok = 2 * (H * (nh + 2 * nkv) * hd + nh * hd * H + 2 * H * I + I * H)
    attn = 4 * nh * hd * T * (T + 1) / 2          # q.k and p.v over the causal triangle
    return L * (per_tok * T + attn) + 2 * H * V     # the head runs for one row


def decode_phase(llm, batch, context, steps, warmup, seed):
    """Fills ``batch`` requests up to (context - steps - warmup) tokens, then times ``steps``
    decode steps on the device.  Returns (ms per step, launches per step, bytes uploaded per step)."""
    import torch
    from pico_vllm_b200 import ops
    from pico_vllm_b200.engine import StepItem
    runner, cache = llm.runner, llm.cache
    V = llm.model.vocab_size
    g = torch.Generator().manual_seed(seed)
    prompt_len = context - steps - warmup
    slots = [cache.acquire(f"bench{i}") for i in range(batch)]
    for s in slots:                                  # prompts in portions of 2048 tokens
        at = 0
        while at < prompt_len:
            n = min(2048, prompt_len - at)
            runner.step([StepItem(s, torch.randint(0, V, (n,), generator=g).tolist(), ())])
            at += n
    toks = torch.randint(0, V, (steps + warmup, batch), generator=g).tolist()
    # every step chooses its tokens (greedy, inside the head's kernel where it can), as a serving step does
    for i in range(warmup):
        runner.step([StepItem(s, [toks[i][j]], (0,)) for j, s in enumerate(slots)], greedy=True)
    torch.cuda.synchronize()
    before = ops.launches
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if PROFILE_RANGE == "decode":
        torch.cuda.profiler.start()
    t0.record()
    for i in range(warmup, warmup + steps):
        logits = runner.step([StepItem(s, [toks[i][j]], (0,)) for j, s in enumerate(slots)], greedy=True)
        if logits is not None:                       # more rows than the head's kernel chooses among: the sampling kernel
            llm.sampler.sample_async(logits, [0.0] * batch, [1.0] * batch, None, out=runner.feedback)
    t1.record()
    torch.cuda.synchronize()
    if PROFILE_RANGE == "decode":
        torch.cuda.profiler.stop()
    ms = t0.elapsed_time(t1) / steps
    launches = (ops.launches - before) / steps
    for s in slots:
        cache.release(s)
    return ms, launches


def e2e_phase(llm, batch, context, steps, warmup, seed):
    """The same decode steps through LLM.submit / LLM.step: host ids in, sampled host ids out."""
    import torch
    V = llm.model.vocab_size
    g = torch.Generator().manual_seed(seed)
    prompt_len = context - steps - warmup
    for _ in range(batch):
        llm.submit(torch.randint(0, V, (prompt_len,), generator=g).tolist(), max_new_tokens=steps + warmup + 64,
                   temperature=0.0, top_p=1.0, ignore_eos=True)
    while any(not r.is_decoding for r in llm.scheduler.running) or llm.scheduler.waiting:
        llm.step()                                    # prompts, in portions
    for _ in range(warmup - 1):
        llm.step()
    torch.cuda.synchronize()
    t_start = time.perf_counter()
    n = 0
    for _ in range(steps):
        llm.step()
        n += 1
    torch.cuda.synchronize()
    dt = time.perf_counter() - t_start
    while llm.scheduler.has_work():
        llm.step()
    return dt * 1000.0 / n


def prefill_phase(llm, T, reps, seed):
    import torch
    from pico_vllm_b200.engine import StepItem
    runner, cache = llm.runner, llm.cache
    V = llm.model.vocab_size
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, V, (T,), generator=g).tolist()
    times = []
    for i in range(reps + 3):
        s = cache.acquire("prefill")
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if PROFILE_RANGE == "prefill" and i == reps + 2:
            torch.cuda.profiler.start()
        t0.record()
        runner.step([StepItem(s, ids, (T - 1,))])
        t1.record()
        torch.cuda.synchronize()
        if PROFILE_RANGE == "prefill" and i == reps + 2:
            torch.cuda.profiler.stop()
        if i >= 3:
            times.append(t0.elapsed_time(t1))
        cache.release(s)
    times.sort()
    return times[len(times) // 2]


def run_micro(args):
    """Single kernels replayed from a CUDA graph over operands larger than L2 (rotating copies of
    the weights, or the caches of many layers), timed with CUDA events: the figures that the
    summaries under profiles/ quote beside the profiler's.  Prints one JSON line."""
    import math
    import torch
    import pico_vllm_b200  # noqa: F401
    from pico_vllm_b200 import ops
    dev = "cuda:0"
    M = args.batch

    def graph_time(fns):
        for f in fns[:3]:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            best = min(best, a.elapsed_time(b) * 1000 / len(fns))
        return best

    out = {"micro": True, "tokens": M, "context": args.context}
    shapes = {"qkv": (2048, 1536), "o": (1536, 1536), "gate_up": (17920, 1536), "down": (1536, 8960),
              "head": (151936, 1536)}
    for name, (N, K) in shapes.items():
        if M > 16:
            break               # the small-batch kernels take at most 16 tokens
        mb = N * K * 2 / 1e6
        copies = max(2, int(600 / mb) + 1)
        ws = [(torch.randn(N, K, device=dev) / math.sqrt(K)).bfloat16() for _ in range(copies)]
        x = torch.randn(M, K, device=dev).bfloat16()
        res = torch.zeros(M, N, device=dev)
        if name == "gate_up":
            mk = lambda w: (lambda: ops.skinny_gate_up_swiglu(x, w))
        elif name in ("o", "down"):
            mk = lambda w: (lambda: ops.skinny_linear_residual(x, w, res))
        elif name == "head":
            mk = lambda w: (lambda: ops.skinny_linear(x, w, None, torch.float32))
        else:
            mk = lambda w: (lambda: ops.skinny_linear(x, w))
        t = graph_time([mk(w) for w in ws] * 2)
        tc = graph_time([(lambda w=w: torch.mm(x, w.t())) for w in ws] * 2)
        out[f"skinny_{name}"] = {"us": round(t, 1), "GBps": round(mb / t * 1e3), "cublas_us": round(tc, 1)}
        del ws
    if M >= 128:                # many tokens: the tcgen05 products against the library's
        for name, (N, K) in shapes.items():
            if name == "head":
                continue
            x = torch.randn(M, K, device=dev).bfloat16()
            w = (torch.randn(N, K, device=dev) / math.sqrt(K)).bfloat16()
            fl = 2.0 * M * N * K
            if name == "gate_up":
                t = graph_time([lambda: ops.tc_gate_up_swiglu(x, w)] * 8)
            else:
                t = graph_time([lambda: ops.tc_linear(x, w)] * 8)
            tc = graph_time([lambda: torch.mm(x, w.t())] * 8)
            out[f"tcgen05_{name}"] = {"us": round(t, 1), "tflops": round(fl / t / 1e6),
                                      "cublas_us": round(tc, 1), "fused": "swiglu" if name == "gate_up" else None}
        # causal attention of one prompt of M tokens over its own pages
        nh, nkv, hd, ps = 12, 2, 128, 16
        blocks = (M + ps - 1) // ps
        k = torch.randn(blocks, nkv, ps, hd, device=dev).bfloat16()
        v = torch.randn(blocks, nkv, ps, hd, device=dev).bfloat16()
        table = torch.randperm(blocks, device=dev).int().view(1, blocks).contiguous()
        q = torch.randn(M, (nh + 2 * nkv) * hd, device=dev).bfloat16()
        o = torch.empty(M, nh * hd, device=dev).bfloat16()
        seg = torch.zeros(M, device=dev).int()
        pos = torch.arange(M, device=dev).int()
        cu = torch.tensor([0, M], device=dev).int()
        pf = torch.zeros(1, device=dev).int()
        dec = torch.zeros(0, device=dev).int()
        maps = (ops.make_kv_tensor_map(k), ops.make_kv_tensor_map(v), ops.make_kv_tensor_map_2d(k),
                ops.make_kv_tensor_map_2d(v, values=True))
        t = graph_time([lambda: ops.paged_attention_mma(q, k, v, o, seg, pos, table, cu, pf, 1, M, dec, 0, nh, nkv, hd,
                                                        ps, None, hd ** -0.5, 1, None, *maps)] * 8)
        fl = 2.0 * 2 * nh * hd * M * (M + 1) / 2          # the visible (query, key) pairs only
        out["prefill_attention"] = {"us": round(t, 1), "tflops_causal": round(fl / t / 1e6)}
        if M <= 4096:
            # the same M tokens as a portion after 14,336 others: with two blocks per query tile, and with one
            ctx = 14336
            blocks = (ctx + M + ps - 1) // ps
            k = torch.randn(blocks, nkv, ps, hd, device=dev).bfloat16()
            v = torch.randn(blocks, nkv, ps, hd, device=dev).bfloat16()
            table = torch.randperm(blocks, device=dev).int().view(1, blocks).contiguous()
            pos = torch.arange(ctx, ctx + M, device=dev).int()
            maps = (ops.make_kv_tensor_map(k), ops.make_kv_tensor_map(v), ops.make_kv_tensor_map_2d(k),
                    ops.make_kv_tensor_map_2d(v, values=True))
            scratch = torch.empty(ops.attention_scratch_floats(M, nh, hd, 2), dtype=torch.float32, device=dev)
            t1 = graph_time([lambda: ops.paged_attention_mma(q, k, v, o, seg, pos, table, cu, pf, 1, M, dec, 0, nh, nkv,
                                                             hd, ps, None, hd ** -0.5, 1, None, *maps)] * 4)
            t2 = graph_time([lambda: ops.paged_attention_mma(q, k, v, o, seg, pos, table, cu, pf, 1, M, dec, 0, nh, nkv,
                                                             hd, ps, None, hd ** -0.5, 1, scratch, *maps,
                                                             pair_min_keys=6144)] * 4)
            out["prefill_attention_after_14336"] = {"us": round(t2, 1), "one_block_per_tile_us": round(t1, 1)}
        print(json.dumps(out))
        return 0
    nh, nkv, hd, ps, L, ctx = 12, 2, 128, 16, 24, args.context
    blocks = ctx // ps
    pages = M * blocks
    k = torch.randn(L, pages, nkv, ps, hd, device=dev).bfloat16()
    v = torch.randn(L, pages, nkv, ps, hd, device=dev).bfloat16()
    table = torch.randperm(pages, device=dev).int().view(M, blocks).contiguous()
    q = torch.randn(M, nh * hd, device=dev).bfloat16()
    seg = torch.arange(M, device=dev).int()
    pos = torch.full((M,), ctx - 1, device=dev).int()
    cu = torch.arange(M + 1, device=dev).int()
    o = torch.empty(M, nh * hd, device=dev).bfloat16()
    maps = [(ops.make_kv_tensor_map(k[l]), ops.make_kv_tensor_map(v[l])) for l in range(L)]
    mb = M * ctx * nkv * hd * 2 * 2 / 1e6
    want = 16 if M * nkv * 16 <= 148 else min(296 // (M * nkv), 8)
    want = max(1, min(want, ctx // 128))
    best_splits = 1
    while best_splits * 2 <= want:
        best_splits *= 2
    for splits in sorted({best_splits, max(1, best_splits // 2)}):
        scratch = torch.empty(max(1, ops.attention_scratch_floats(M, nh, hd, splits)), device=dev)
        t = graph_time([(lambda l=l: ops.paged_attention_mma(q, k[l], v[l], o, seg, pos, table, cu, None, 0, 0, None, M,
                                                             nh, nkv, hd, ps, None, 1 / math.sqrt(hd), splits, scratch,
                                                             *maps[l])) for l in range(L)])
        out[f"decode_attention_splits{splits}"] = {"us": round(t, 1), "GBps": round(mb / t * 1e3), "MB": round(mb, 1)}
    print(json.dumps(out))
    return 0


def random_model_on_device(raw, device="cuda:0", seed=0):
    """A model of the given configuration with random weights drawn on the device (the larger shapes: drawing
    7.6 G normal numbers on the host and writing them to a folder would take minutes); bfloat16 matrices, float32
    vectors, N(0, 0.02) and 1 + N(0, 0.02) for norm weights, as the random-weights mode writes them."""
    import torch
    from pico_vllm_b200.engine.core import _prepare_precision
    from pico_vllm_b200.registry import build_model, config_from_dict
    cfg = config_from_dict(raw)
    model = build_model(cfg)
    _prepare_precision("bfloat16")
    g = torch.Generator(device=device).manual_seed(seed)
    for b in model.bindings:
        for p in b.part.params():
            t = torch.randn(p.shape, generator=g, device=device, dtype=torch.float32) * 0.02
            if p.init == "one_plus_normal":
                t = t + 1.0
            b.part.assign(p.attr, t if p.kind == "vector" else t.to(torch.bfloat16))
    model.materialize(device, torch.bfloat16)
    return cfg, model


def step_flops(cfg, q_lens, starts):
    """Floating-point operations of one step: the products of every token, attention over each token's visible
    keys, and the head for one row per segment."""
    H, I, V, L = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers
    nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    per_tok = 2 * (H * (nh + 2 * nkv) * hd + nh * hd * H + 2 * H * I + I * H)
    attn = sum(4 * nh * hd * (n * st + n * (n + 1) / 2) for n, st in zip(q_lens, starts))
    return L * (per_tok * sum(q_lens) + attn) + 2 * H * V * len(q_lens)


def run_shape(args):
    """The two larger shapes of the architecture with the workloads named for them: 3b - continuous batching of
    32 requests (prompts of 64 to 2,048 tokens, 128 generated tokens each) through ``LLM.generate``; 7b - decode
    steps of 64 requests at context 8,192, and steps that hold one 2,048-token portion of a prompt beside 63
    decoding requests.  Prints one JSON line."""
    import torch
    import pico_vllm_b200  # noqa: F401
    from pico_vllm_b200 import LLM, SamplingParams, ops
    from pico_vllm_b200.engine import StepItem
    pk = peaks()
    name, raw = SHAPES[args.config]
    raw = dict(raw, num_hidden_layers=args.layers or raw["num_hidden_layers"])
    t0 = time.time()
    cfg, model = random_model_on_device(raw)
    print(f"[bench] {name}: random weights on the device in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    out = {"impl": "ours", "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)",
           "config": {"model": name, "layers": cfg.num_hidden_layers, "layers_full": SHAPES[args.config][1]["num_hidden_layers"],
                      "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                      "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                      "tied": cfg.tie_word_embeddings, "page_size": 16, "peaks": pk["source"]}}
    sampler = ClockSampler()
    if args.config == "3b":
        n_req, n_new = 32, 128
        llm = LLM(model, dtype="bfloat16", page_size=16, num_pages=n_req * ((2048 + n_new) // 16 + 2), max_num_seqs=n_req,
                  max_num_batched_tokens=4096, prefill_chunk=2048, max_model_len=2048 + n_new + 16)
        wbytes = weight_bytes(llm.model)
        sp = SamplingParams(temperature=0.0, max_new_tokens=n_new, ignore_eos=True)

        def workload(seed):
            g = torch.Generator().manual_seed(seed)
            lens = torch.randint(64, 2049, (n_req,), generator=g).tolist()
            return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
        llm.generate(workload(1), sp)                        # the same workload once before: graphs recorded, libraries warm
        prompts = workload(2)
        steps0 = llm.stats["steps"]
        torch.cuda.synchronize()
        sampler.start()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        clocks = sampler.stop()
        steps = llm.stats["steps"] - steps0
        n_prompt = sum(len(p) for p in prompts)
        assert all(len(o.token_ids) == n_new for o in outs)
        out.update({"metric": f"generated tok/s end to end ({name}, {n_req} requests, prompts 64..2048, {n_new} new tokens each)",
                    "value": round(n_req * n_new / dt, 1), "unit": "tok/s", "seconds": round(dt, 4), "steps": steps,
                    "prompt_tokens": n_prompt, "all_tokens_per_s": round((n_prompt + n_req * n_new) / dt, 1),
                    "ms_per_step": round(dt * 1000.0 / steps, 4), "preemptions": llm.scheduler.num_preemptions,
                    # every step reads every weight at least once: a lower bound of the bytes moved
                    "roofline": {"bound": "hbm", "achieved": round(steps * wbytes / dt / 1e9, 1), "peak": pk["hbm_gbs"],
                                 "unit": "GB/s", "frac": round(steps * wbytes / dt / 1e9 / pk["hbm_gbs"], 4),
                                 "note": "weights only, once per step"},
                    "clocks": clocks})
    else:
        batch, context = args.batch or 64, args.context or 8192
        llm = LLM(model, dtype="bfloat16", page_size=16, num_pages=max(batch, 64) * ((context + 2048 + 128) // 16 + 1) + 64,
                  max_num_seqs=max(batch, 64), max_num_batched_tokens=4096, prefill_chunk=2048, max_model_len=context + 6 * 2048)
        wbytes = weight_bytes(llm.model)
        kvb = kv_bytes_per_token(llm.model, llm.cache)
        sampler.start()
        ms, launches = decode_phase(llm, batch, context, args.steps, args.warmup, seed=1)
        clocks = sampler.stop()
        step_bytes = wbytes + batch * (context - args.steps / 2) * kvb
        # one 2,048-token portion of a prompt beside 63 decoding requests at context 8,192
        runner, cache = llm.runner, llm.cache
        g = torch.Generator().manual_seed(5)
        V = cfg.vocab_size
        slots = [cache.acquire(f"d{i}") for i in range(63)]
        for s_ in slots:
            for at in range(0, context - 64, 2048):
                n = min(2048, context - 64 - at)
                runner.step([StepItem(s_, torch.randint(0, V, (n,), generator=g).tolist(), ())])
        big = cache.acquire("p")
        times, fl = [], 0.0
        for rep in range(5):
            items = [StepItem(big, torch.randint(0, V, (2048,), generator=g).tolist(), (2047,))]
            items += [StepItem(s_, [int(torch.randint(0, V, (1,), generator=g))], (0,)) for s_ in slots]
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            runner.step(items)
            b.record()
            torch.cuda.synchronize()
            if rep >= 2:
                times.append(a.elapsed_time(b))
                fl = step_flops(cfg, [2048] + [1] * 63, [rep * 2048] + [context - 64 + rep] * 63)
        times.sort()
        mixed_ms = times[len(times) // 2]
        out.update({"metric": f"decode tok/s ({name}, batch {batch}, context {context})",
                    "value": round(batch / ms * 1000.0, 1), "unit": "tok/s", "steps": args.steps, "warmup": args.warmup,
                    "ms_per_step": round(ms, 4), "launches_per_step": round(launches, 1),
                    "roofline": {"bound": "hbm", "achieved": round(step_bytes / (ms / 1e3) / 1e9, 1), "peak": pk["hbm_gbs"],
                                 "unit": "GB/s", "frac": round(step_bytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)},
                    "mixed": {"what": "one 2,048-token portion beside 63 decoding requests at context 8,192",
                              "ms_per_step": round(mixed_ms, 3), "tokens_per_s": round((2048 + 63) / mixed_ms * 1e3, 1),
                              "frac": round(fl / (mixed_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4), "bound": "bf16 tensor"},
                    "clocks": clocks})
    print(json.dumps(out))
    return 0


def run_ours(args):
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: bench.py needs a GPU"}))
        return 1
    import pico_vllm_b200  # noqa: F401
    from pico_vllm_b200 import LLM, ops
    pk = peaks()
    batch, context = args.batch, args.context
    layers = args.layers
    tmp = tempfile.mkdtemp(prefix="pico_bench_", dir=scratch_dir(4 << 30))
    try:
        cfg = make_model_folder(layers, tmp)
        max_b = max(64, batch) if not args.no_points else batch
        longest = max(context, 512 + 8 + 256, 2048) + 128     # the decode runs, the 512 + 256 workload, the 2,048-token prompt
        pages = max_b * ((max(context, 512 + 8 + 256) + 128) // 16 + 1) + 256
        llm = LLM(tmp, dtype="bfloat16", page_size=16, num_pages=pages, max_num_seqs=max_b,
                  max_num_batched_tokens=4096, prefill_chunk=2048, max_model_len=longest,
                  use_cuda_graph=True)
    finally:
        for f in os.listdir(tmp):
            os.remove(os.path.join(tmp, f))
        os.rmdir(tmp)
    wbytes = weight_bytes(llm.model)
    kvb = kv_bytes_per_token(llm.model, llm.cache)

    T = 2048
    if args.only == "prefill":
        pre_ms = prefill_phase(llm, T, reps=2, seed=3)
        print(json.dumps({"only": "prefill", "tokens": T, "ms": round(pre_ms, 3), "layers": layers}))
        return 0
    sampler = ClockSampler()
    sampler.start()
    ms, launches = decode_phase(llm, batch, context, args.steps, args.warmup, seed=1)
    clocks = sampler.stop()
    if args.only == "decode":
        print(json.dumps({"only": "decode", "batch": batch, "context": context, "ms_per_step": round(ms, 4),
                          "launches_per_step": launches, "layers": layers}))
        return 0

    e2e_ms = e2e_phase(llm, batch, context, args.steps, args.warmup, seed=2)
    pre_ms = prefill_phase(llm, T, reps=5, seed=3)
    def frac(b, ctx_mid, step_ms):
        return round((wbytes + b * ctx_mid * kvb) / (step_ms / 1000.0) / 1e9 / pk["hbm_gbs"], 4)

    points = {}
    if not args.no_points:
        for b in (1, 64):
            pms, _ = decode_phase(llm, b, context, 32, 8, seed=10 + b)
            points[f"decode_b{b}"] = round(b / pms * 1000.0, 1)
            points[f"decode_b{b}_ms"] = round(pms, 4)
            points[f"decode_b{b}_frac"] = frac(b, context - 16, pms)
        # the reference's own decode workload: a 512-token prompt, then 256 generated tokens (the 256 steps are timed)
        for b in (1, 8, 64):
            pms, _ = decode_phase(llm, b, 512 + 8 + 256, 256, 8, seed=20 + b)
            points[f"gen256_b{b}"] = round(b / pms * 1000.0, 1)
            points[f"gen256_b{b}_ms"] = round(pms, 4)
            points[f"gen256_b{b}_frac"] = frac(b, 512 + 8 + 128, pms)

    step_bytes = wbytes + batch * (context - args.steps / 2) * kvb
    achieved = step_bytes / (ms / 1000.0) / 1e9
    flops = prefill_flops(cfg, T)
    pre_frac = flops / (pre_ms / 1000.0) / (pk["bf16_tflops"] * 1e12)
    value = batch / ms * 1000.0
    bucket = llm.runner._bucket(batch)
    stage = max(e["buffers"].host.numel() for k, e in llm.runner._graphs.items() if k[:2] == ("decode", bucket)) * 4
    out = {
        "metric": f"decode tok/s (Qwen2.5-1.5B shape, batch {batch}, context {context})",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)",
        "impl": "ours",
        "config": {"model": "Qwen2.5-1.5B shape", "layers": layers, "layers_full": FULL_LAYERS,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied": cfg.tie_word_embeddings, "global_batch": batch, "seq_len": context,
                   "page_size": 16, "parallelism": "single GPU", "cuda_graph": True, "sampling": "greedy, in the head's kernel",
                   "l2": "no flush: each step reads >3 GB of weights and cache, L2 is 126 MB",
                   "peaks": pk["source"]},
        "clocks": clocks,
        "e2e": {"value": round(batch / e2e_ms * 1000.0, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": stage, "d2h_bytes_per_step": 4 * batch},
        "gpu_launches": int(round(launches * args.steps)),
        "launches_per_step": round(launches, 1),
        "prefill": {"value": round(T / pre_ms * 1000.0, 1), "tokens": T, "ms": round(pre_ms, 3),
                    "frac": round(pre_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "decode_b1_vs_published_97": (round(points["decode_b1"] / PUBLISHED_DECODE_B1, 2)
                                      if "decode_b1" in points else None),
    }
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="decoding requests (default 8; 64 for --config 7b)")
    ap.add_argument("--context", type=int, default=None, help="context length of the decode steps (default 4096; 8192 for --config 7b)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the full model (named in config)")
    ap.add_argument("--config", choices=sorted(SHAPES), default="1.5b",
                    help="1.5b: the default run; 3b, 7b: the larger shapes with the workloads named for them")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one phase only and print a short line (for profiling; not a bench value)")
    ap.add_argument("--micro", action="store_true",
                    help="time single decode kernels replayed from a graph (skinny products, decode attention)")
    ap.add_argument("--profile-range", choices=["decode", "prefill"], default=None,
                    help="bracket that phase's timed region with cudaProfilerStart/Stop (ncu --profile-from-start off)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported (this engine runs on a single GPU)")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.config == "1.5b" or args.micro:
        args.layers = args.layers or FULL_LAYERS
        args.batch = args.batch or 8
        args.context = args.context or 4096
    if args.impl == "reference" and args.config != "1.5b":
        print(json.dumps({"impl": "reference", "unavailable": "the reference has the Qwen2.5-1.5B shape only "
                                                              "(pico_vllm/model.py:15-26)"}))
        return 0
    if args.impl == "reference":
        # the unmodified reference from baseline/_ref through its own Engine.submit / Engine.step; nothing of this
        # repository's package is imported on that path
        from baseline.reference_arm import run as run_reference
        from types import SimpleNamespace

        def flops(T, layers):
            shape = SimpleNamespace(hidden_size=MODEL["hidden_size"], intermediate_size=MODEL["intermediate_size"],
                                    vocab_size=MODEL["vocab_size"], num_hidden_layers=layers,
                                    num_attention_heads=MODEL["num_attention_heads"],
                                    num_key_value_heads=MODEL["num_key_value_heads"],
                                    head_dim=MODEL["hidden_size"] // MODEL["num_attention_heads"])
            return prefill_flops(shape, T)
        return run_reference(args, peaks(), ClockSampler(), flops, PUBLISHED_DECODE_B1)
    global PROFILE_RANGE
    PROFILE_RANGE = args.profile_range
    if args.only:
        args.no_points = True
    if args.micro:
        return run_micro(args)
    if args.config != "1.5b":
        return run_shape(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
