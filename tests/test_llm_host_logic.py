"""The entry point, scheduler and sampler wiring on the CPU with kernel doubles."""
import torch

import fake_ops
import helpers
import plain_qwen2 as plain


def _llm(monkeypatch, tmp_path, name, **opts):
    fake_ops.install(monkeypatch)
    from pico_vllm_b200 import LLM
    helpers.write_tiny_model(name, tmp_path, dtype="float32")
    return LLM(str(tmp_path), dtype="float32", device="cpu", use_cuda_graph=False,
               page_size=helpers.TINY[name]["page_size"], **opts)


import pytest


@pytest.mark.parametrize("ahead", [True, False])
def test_greedy_generation_equals_plain(monkeypatch, tmp_path, ahead):
    from pico_vllm_b200 import SamplingParams
    llm = _llm(monkeypatch, tmp_path, "a", max_cache_tokens=512, async_scheduling=ahead)
    cfg = helpers.tiny_config("a")
    prompts = [helpers.random_ids(n, cfg.vocab_size, 7 + n) for n in (5, 17, 33)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True))
    tensors = helpers.tiny_tensors("a", torch.float32)
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain.greedy_generate(p, tensors, helpers.plain_config(cfg), 8)
        assert o.finish_reason == "length"
    llm.cache.check()
    assert all(g.pool.in_use == 0 for g in llm.cache.groups)


def test_chunked_prefill_with_preemption_gives_the_same_tokens(monkeypatch, tmp_path):
    from pico_vllm_b200 import SamplingParams
    # 9 requests, few pages, portions of 7 tokens: requests are pre-empted and recomputed
    llm = _llm(monkeypatch, tmp_path, "b", num_pages=14, max_num_seqs=4, max_num_batched_tokens=16,
               prefill_chunk=7, max_model_len=112)
    cfg = helpers.tiny_config("b")
    prompts = [helpers.random_ids(n, cfg.vocab_size, 50 + n) for n in (1, 9, 24, 40, 13, 30, 6, 21, 35)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=10, ignore_eos=True))
    tensors = helpers.tiny_tensors("b", torch.float32)
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain.greedy_generate(p, tensors, helpers.plain_config(cfg), 10)
    assert llm.scheduler.num_preemptions > 0
    llm.cache.check()


def test_submit_step_calls_of_the_reference(monkeypatch, tmp_path):
    llm = _llm(monkeypatch, tmp_path, "a", max_cache_tokens=256)
    a = llm.submit([1, 2, 3], max_new_tokens=3, temperature=0, top_p=1.0, ignore_eos=True)
    b = llm.submit([4, 5], max_new_tokens=5, temperature=0.8, top_p=0.9, seed=3, ignore_eos=True)
    llm.mark_finished()
    assert llm.submit([1], 1, 0, 1.0) == -1
    got = {}
    while not llm.is_done():
        for rid, ids in llm.step():
            got[rid] = ids
    assert len(got[a]) == 3 + 3 and got[a][:3] == [1, 2, 3]
    assert len(got[b]) == 2 + 5


def test_sampled_tokens_do_not_depend_on_batching(monkeypatch, tmp_path):
    from pico_vllm_b200 import SamplingParams
    llm = _llm(monkeypatch, tmp_path, "a", max_cache_tokens=512)
    cfg = helpers.tiny_config("a")
    prompts = [helpers.random_ids(n, cfg.vocab_size, 90 + n) for n in (4, 11, 19)]
    sp = SamplingParams(temperature=0.8, top_p=0.95, max_new_tokens=6, seed=11, ignore_eos=True)
    together = llm.generate(prompts, sp)
    # the same request ids (0, 1, 2) one at a time in a fresh engine
    llm2 = _llm(monkeypatch, tmp_path, "a", max_cache_tokens=512)
    alone = [llm2.generate([p], sp)[0] for p in prompts]
    assert [o.token_ids for o in together] == [o.token_ids for o in alone]


@pytest.mark.parametrize("ahead", [True, False])
def test_end_token_stops_a_request_and_frees_its_pages(monkeypatch, tmp_path, ahead):
    from pico_vllm_b200 import SamplingParams
    cfg = helpers.tiny_config("a")
    prompts = [helpers.random_ids(n, cfg.vocab_size, 7 + n) for n in (5, 17, 33)]
    tensors = helpers.tiny_tensors("a", torch.float32)
    want = [plain.greedy_generate(p, tensors, helpers.plain_config(cfg), 10) for p in prompts]
    eos = want[1][3]                      # request 1 meets it as its 4th token
    llm = _llm(monkeypatch, tmp_path, "a", max_cache_tokens=512, async_scheduling=ahead)
    llm.scheduler.eos_token_id = eos
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=10))
    for w, o in zip(want, outs):
        cut = w.index(eos) + 1 if eos in w else len(w)
        assert o.token_ids == w[:cut]
        assert o.finish_reason == ("eos" if eos in w else "length")
    llm.cache.check()
    assert all(g.pool.in_use == 0 for g in llm.cache.groups) and llm.cache.free_slots == llm.cache.max_num_seqs
    # the engine can go on after that
    again = llm.generate(prompts[:1], SamplingParams(temperature=0.0, max_new_tokens=10, ignore_eos=True))
    assert again[0].token_ids == want[0]


@pytest.mark.parametrize("ahead", [True, False])
def test_pages_held_by_a_request_in_flight_are_waited_for(monkeypatch, tmp_path, ahead):
    """4 pages: a request that fills 3 of them and generates a page's worth of tokens, then a
    short one.  One step ahead of the device, the first request's last token is still in flight
    (and its pages are still held) when the second is scheduled: the scheduler must wait for that
    step instead of reporting that the second request does not fit even alone."""
    from pico_vllm_b200 import SamplingParams
    ps = helpers.TINY["a"]["page_size"]
    llm = _llm(monkeypatch, tmp_path, "a", num_pages=4, max_num_seqs=2, async_scheduling=ahead)
    cfg = helpers.tiny_config("a")
    prompts = [helpers.random_ids(3 * ps, cfg.vocab_size, 1), helpers.random_ids(ps + 3, cfg.vocab_size, 2)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=ps, ignore_eos=True))
    tensors = helpers.tiny_tensors("a", torch.float32)
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain.greedy_generate(p, tensors, helpers.plain_config(cfg), ps)
    llm.cache.check()
    assert all(g.pool.in_use == 0 for g in llm.cache.groups)


def test_a_bounded_wait_that_ran_out_is_an_error_not_tokens(monkeypatch, tmp_path):
    """The kernels' waits are bounded; a wait that runs out leaves a status word set and part of a result
    unwritten.  The entry point reads the words before tokens leave it (when a request completes)."""
    from pico_vllm_b200 import SamplingParams, ops
    from pico_vllm_b200.errors import KernelError
    llm = _llm(monkeypatch, tmp_path, "a", max_cache_tokens=256)
    monkeypatch.setattr(ops, "_lib", object())          # as if the library were loaded
    for name in ("tma_status", "tca_status", "tc_status"):
        monkeypatch.setattr(ops, name, lambda: 0)
    outs = llm.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_new_tokens=2, ignore_eos=True))
    assert len(outs[0].token_ids) == 2
    monkeypatch.setattr(ops, "tca_status", lambda: 1)
    with pytest.raises(KernelError, match="paged_prefill_tcgen05"):
        llm.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_new_tokens=2, ignore_eos=True))


def test_prompt_token_ids_outside_the_vocabulary_are_refused(monkeypatch, tmp_path):
    from pico_vllm_b200 import SamplingParams
    from pico_vllm_b200.errors import ConfigError
    llm = _llm(monkeypatch, tmp_path, "a", max_cache_tokens=256)
    vocab = helpers.tiny_config("a").vocab_size
    for bad in ([1, -3], [1, vocab]):
        with pytest.raises(ConfigError, match="prompt token ids"):
            llm.generate([bad], SamplingParams(max_new_tokens=2))
    assert not llm.scheduler.has_work()
