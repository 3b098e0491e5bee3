"""Command line, in the manner of the reference's entry script.

``python -m pico_vllm_b200.cli run --model DIR --prompt-ids 1,2,3`` does what the reference's
``run_single.py`` does with its inline constants (pico_vllm/run_single.py:10-37): load the model
folder, make a cache of ``--num-gpu-blocks`` (500) pages of ``--block-size`` (16) tokens, submit
one prompt with ``--max-new-tokens`` (20), ``--temperature`` (0 = greedy) and ``--top-p`` (1.0),
step until it completes and print ``[request id] output``.  Option names are the reference's
argument names (num_gpu_blocks, block_size, max_new_tokens, temperature, top_p, use_cuda_graph,
max_batch_size -> here the largest graph batch, max_num_seqs); options it has no name for
(dtype, token budget, portion size, seed) are additions.

``python -m pico_vllm_b200.cli random-model --config CONFIG.json --seed S --out DIR`` writes a
model folder with random weights (config.json, model.safetensors) from a configuration.
"""
from __future__ import annotations

import argparse
import json
import sys


def _run(args) -> int:
    from . import LLM
    from .config import EngineConfig
    buckets = tuple(b for b in (1, 2, 4, 8, 16, 32, 64, 128, 256) if b < args.max_batch_size) + (args.max_batch_size,)
    cfg = EngineConfig(dtype=args.dtype, page_size=args.block_size, num_pages=args.num_gpu_blocks,
                       max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
                       prefill_chunk=args.prefill_chunk, max_model_len=args.max_model_len,
                       use_cuda_graph=args.use_cuda_graph, graph_batch_sizes=buckets, seed=args.seed,
                       device=args.device)
    llm = LLM(args.model, engine_config=cfg)
    prompts = []
    for p in args.prompt or []:
        prompts.append(p)
    for p in args.prompt_ids or []:
        prompts.append([int(t) for t in p.replace(" ", "").split(",") if t])
    if not prompts:
        print("give at least one --prompt TEXT or --prompt-ids 1,2,3", file=sys.stderr)
        return 2
    for p in prompts:
        llm.submit(p, max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_p=args.top_p,
                   seed=args.seed, ignore_eos=args.ignore_eos)
    llm.mark_finished()
    while not llm.is_done():
        for rid, out in llm.step():
            print(f"[{rid}] {out if isinstance(out, str) else ' '.join(str(t) for t in out)}", flush=True)
    return 0


def _random_model(args) -> int:
    from .registry import config_from_dict
    from .weights import write_random_model
    with open(args.config, "r", encoding="utf-8") as f:
        raw = json.load(f)
    cfg = config_from_dict(raw, where=args.config)
    write_random_model(cfg, args.seed, args.out, dtype=args.dtype, std=args.std)
    print(f"wrote {args.out}/config.json and {args.out}/model.safetensors")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pico_vllm_b200.cli", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    run = sub.add_parser("run", help="generate from prompts")
    run.add_argument("--model", "--weights", dest="model", default="./weights",
                     help="model folder (the reference reads ./weights)")
    run.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    run.add_argument("--prompt", action="append", help="text prompt (needs a tokenizer in the folder)")
    run.add_argument("--prompt-ids", action="append", help="prompt as comma-separated token ids")
    run.add_argument("--max-new-tokens", type=int, default=20)
    run.add_argument("--temperature", type=float, default=0.0)
    run.add_argument("--top-p", type=float, default=1.0)
    run.add_argument("--seed", type=int, default=0)
    run.add_argument("--ignore-eos", action="store_true")
    run.add_argument("--num-gpu-blocks", type=int, default=500)
    run.add_argument("--block-size", type=int, default=16)
    run.add_argument("--max-num-seqs", type=int, default=4)
    run.add_argument("--max-batch-size", type=int, default=8, help="largest decode batch replayed from a CUDA graph")
    run.add_argument("--max-num-batched-tokens", type=int, default=2048)
    run.add_argument("--prefill-chunk", type=int, default=None)
    run.add_argument("--max-model-len", type=int, default=None)
    run.add_argument("--use-cuda-graph", dest="use_cuda_graph", action="store_true", default=True)
    run.add_argument("--no-cuda-graph", dest="use_cuda_graph", action="store_false")
    run.add_argument("--device", default="cuda:0")
    run.set_defaults(fn=_run)
    rnd = sub.add_parser("random-model", help="write a model folder with random weights")
    rnd.add_argument("--config", required=True, help="a config.json of a supported architecture")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    rnd.add_argument("--std", type=float, default=0.02)
    rnd.set_defaults(fn=_random_model)
    args = ap.parse_args(argv)
    from .errors import PicoError
    try:
        return args.fn(args)
    except PicoError as e:          # what the engine refuses on purpose: one line, no traceback
        print(f"{type(e).__name__}: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
