"""bin/trace_run as a user runs it: a model folder, steps on standard input, logits in files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REL = {"float32": 5e-5, "bfloat16": 3e-2}


def _run(model_dir, out_dir, dtype, steps, max_tokens):
    lines = "".join(json.dumps(dict(step=i, **st)) + "\n" for i, st in enumerate(steps))
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(model_dir),
                        "--dtype", dtype, "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                       input=lines, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_trace_run_mixed_with_page_reuse(tmp_path, dtype, name):
    cfg = helpers.tiny_config(name)
    model_dir = helpers.write_tiny_model(name, tmp_path / "model", dtype=dtype)
    reqs = {f"r{i}": helpers.random_ids(n, cfg.vocab_size, 300 + i) for i, n in enumerate([40, 7, 95, 33, 64, 130])}
    steps = helpers.trace_mixed(reqs, max_live=4, seed=1) + helpers.trace_tail_decode({"t": reqs["r2"]}, 32)
    _run(model_dir, tmp_path / "out", dtype, steps, helpers.live_token_peak(steps))
    tensors = helpers.tiny_tensors(name, torch.float32 if dtype == "float32" else torch.bfloat16)
    reqs["t"] = reqs["r2"]
    logits = {rid: plain.forward(ids, tensors, helpers.plain_config(cfg)) for rid, ids in reqs.items()}
    want = helpers.expected_logits(steps, reqs, logits)
    for i, w in enumerate(want):
        path = tmp_path / "out" / f"{i}.f32"
        if w is None:
            assert not path.exists()
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(-1, cfg.vocab_size))
        assert got.shape == w.shape
        helpers.assert_close_logits(got, w, REL[dtype], f"step {i}")
