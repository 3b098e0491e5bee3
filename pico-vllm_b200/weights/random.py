"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.  Matrices and biases ~ N(0, std), norm weights 1 + N(0, std), drawn
on the CPU in float32 and stored in ``dtype``.  Every tensor has a generator of its own, keyed
by (seed, index of the tensor in the order of the model's bindings), so tensors can be drawn
in parallel and still depend on nothing but the seed.  The reference has no such mode (it
loads Qwen2.5-1.5B from ./weights, pico_vllm/run_single.py:12)."""
from __future__ import annotations

import json
import os
from concurrent.futures import ThreadPoolExecutor
from typing import Dict

import numpy as np
import torch

from ..registry import build_model


def random_tensors(config, seed: int, std: float = 0.02, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Tensor name -> random tensor for every tensor the architecture's model needs."""
    model = build_model(config)
    jobs = []
    for b in model.bindings:
        for param in b.part.params():
            for piece in param.pieces:
                jobs.append((b.names[piece.key], tuple(piece.shape), param.init))

    def draw(job):
        idx, (name, shape, init) = job
        rng = np.random.Generator(np.random.Philox(np.random.SeedSequence([seed, idx])))
        t = torch.from_numpy(rng.standard_normal(shape, dtype=np.float32)) * std
        if init == "one_plus_normal":
            t = t + 1.0
        return name, t.to(dtype)

    with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as pool:
        return dict(pool.map(draw, enumerate(jobs)))


def write_random_model(config, seed: int, out_dir: str, dtype: str = "bfloat16", std: float = 0.02) -> str:
    """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors``; returns out_dir."""
    from safetensors.torch import save_file
    from ..config.engine import canonical_dtype
    dtype = canonical_dtype(dtype)
    os.makedirs(out_dir, exist_ok=True)
    tensors = random_tensors(config, seed, std, getattr(torch, dtype))
    raw = config.to_dict()
    raw["torch_dtype"] = dtype
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw, f, indent=2)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
    return out_dir
