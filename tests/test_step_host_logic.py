"""The step function, the cache and the batch building on the CPU, with the kernels replaced
by torch doubles (tests/fake_ops.py): every way of cutting requests into steps must give the
plain implementation's logits.  What is tested here is the host side: positions, cache rows,
block tables, page reuse, windows giving pages back, wanted rows."""
import pytest
import torch

import fake_ops
import helpers
import plain_qwen2 as plain

LENGTHS = {"a": [5, 17, 33, 70], "b": [1, 9, 24, 40, 77], "c": [3, 21, 50]}


def _requests(name, vocab):
    return {f"r{i}": helpers.random_ids(n, vocab, 1000 + i) for i, n in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("name", ["a", "b", "c"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_every_cutting_matches_plain(monkeypatch, name, cut):
    fake_ops.install(monkeypatch)
    cfg = helpers.tiny_config(name)
    reqs = _requests(name, cfg.vocab_size)
    steps = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_tail_decode(r, 32),
             "portions": helpers.trace_portions, "mixed": helpers.trace_mixed}[cut](reqs)
    runner, tensors = helpers.make_runner_from_tensors(name, "float32", "cpu", helpers.live_token_peak(steps))
    pcfg = helpers.plain_config(cfg)
    plain_logits = {rid: plain.forward(ids, tensors, pcfg) for rid, ids in reqs.items()}
    want = helpers.expected_logits(steps, reqs, plain_logits)
    got = helpers.replay(runner, steps)
    for i, (g, w) in enumerate(zip(got, want)):
        assert (g is None) == (w is None)
        if w is not None:
            helpers.assert_close_logits(g, w, 2e-5, f"{name}/{cut} step {i}")
    for g in runner.cache.groups:
        assert g.pool.in_use == 0


def test_window_group_gives_pages_back(monkeypatch):
    fake_ops.install(monkeypatch)
    runner, _ = helpers.make_runner_from_tensors("b", "float32", "cpu", 256)
    from pico_vllm_b200.engine import StepItem
    cache = runner.cache
    full = [g for g in cache.groups if g.spec.window is None][0]
    win = [g for g in cache.groups if g.spec.window is not None][0]
    slot = cache.acquire("x")
    runner.step([StepItem(slot, helpers.random_ids(100, 512, 5), ())])
    assert full.pool.in_use == 13                     # ceil(100 / 8)
    # the next query is at position 100 and reads keys 77..100: blocks 0..8 (positions < 72) are dead
    assert win.pool.in_use == 13 - 9
    for _ in range(30):
        runner.step([StepItem(slot, [1], (0,))])
        assert win.pool.in_use <= 4 + 1
    cache.release(slot)
    cache.check()
    assert full.pool.in_use == 0 and win.pool.in_use == 0
