"""The Python entry point.

``LLM`` keeps the reference engine's four calls with their meanings - ``submit(prompt,
max_new_tokens, temperature, top_p) -> request id``, ``step() -> [(request id, output)]`` for
the requests that completed in that step, ``mark_finished()`` (no more requests will come) and
``is_done()`` (pico_vllm/engine.py:243-282, 465-475) - and adds ``generate(prompts, params)``,
which runs a list of prompts to the end.  Prompts are lists of token ids, or text when the model
folder has a tokenizer; a completed request's output is, as in the reference, the prompt and the
generated tokens together (text with a tokenizer, ids without), and ``generate`` returns
``RequestOutput`` objects.  One ``step`` is one batch through the step function: single tokens
of decoding requests beside portions of prompts.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from .. import ops
from ..config.engine import EngineConfig
from ..errors import ConfigError, ScheduleError
from ..sampling import Sampler, SamplingParams, uniform_for
from .core import make_cache, load_model
from .runner import ModelRunner, StepItem
from .scheduler import Request, Scheduler

Prompt = Union[str, Sequence[int]]


@dataclass
class RequestOutput:
    request_id: int
    prompt_token_ids: List[int]
    token_ids: List[int]            # the generated tokens
    text: Optional[str]             # generated text, when the folder has a tokenizer
    finish_reason: Optional[str]
    preemptions: int = 0


class LLM:
    def __init__(self, model: str, dtype: str = "bfloat16", engine_config: Optional[EngineConfig] = None,
                 tokenizer=None, **engine_options):
        """``model``: folder with config.json and safetensors (or a model object that already has its
        weights on the device, as ``engine.load_model`` returns).  ``engine_options`` are fields of
        EngineConfig (page_size, num_pages, max_cache_tokens, max_num_seqs,
        max_num_batched_tokens, prefill_chunk, max_model_len, use_cuda_graph, seed, device)."""
        if engine_config is None:
            engine_config = EngineConfig(dtype=dtype, **engine_options)
        elif engine_options:
            raise ConfigError("give either engine_config or separate engine options, not both")
        self.cfg = engine_config
        self.model = load_model(model, self.cfg) if isinstance(model, (str, os.PathLike)) else model
        self.cache = make_cache(self.model, self.cfg)
        self.runner = ModelRunner(self.model, self.cache, self.cfg)
        self.sampler = Sampler(self.cfg.device, self.cfg.seed)
        self.tokenizer = tokenizer if tokenizer is not None else (
            _maybe_tokenizer(model) if isinstance(model, (str, os.PathLike)) else None)
        eos = getattr(self.model.config, "eos_token_id", None)
        if eos is None and self.tokenizer is not None:
            eos = getattr(self.tokenizer, "eos_token_id", None)
        self.eos_token_id = eos
        self.scheduler = Scheduler(self.cache, self.cfg.max_num_seqs, self.cfg.max_num_batched_tokens,
                                   self.cfg.prefill_chunk, eos)
        self._next_id = 0
        self._no_more = False
        self._pending = None            # (plan, tokens on their way) of the step launched last
        self.requests: Dict[int, Request] = {}
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0}

    # ------------------------------------------------------------------ the reference's four calls
    def submit(self, prompt: Prompt, max_new_tokens: int = 16, temperature: float = 1.0, top_p: float = 1.0,
               seed: Optional[int] = None, ignore_eos: bool = False) -> int:
        """Queues a request; returns its id, or -1 after ``mark_finished`` (pico_vllm/engine.py:250-251)."""
        if self._no_more:
            return -1
        params = SamplingParams(max_new_tokens=max_new_tokens, temperature=temperature, top_p=top_p,
                                seed=seed, ignore_eos=ignore_eos)
        ids = self._encode(prompt)
        rid = self._next_id
        self._next_id += 1
        req = Request(rid, ids, params.max_new_tokens, params.temperature, params.top_p, params.ignore_eos,
                      params.seed)
        self.scheduler.add(req)
        self.requests[rid] = req
        return rid

    def mark_finished(self) -> None:
        self._no_more = True

    def is_done(self) -> bool:
        return self._no_more and not self.scheduler.has_work() and self._pending is None

    def step(self) -> List[Tuple[int, Union[str, List[int]]]]:
        """One batch: schedule, run, sample, finish.  Returns (id, prompt + generated) of the
        requests that completed, as text if there is a tokenizer, else as token ids."""
        return [(r.request_id, self._decode(r.all_ids) if self.tokenizer is not None else r.all_ids)
                for r in self._step()]

    # ------------------------------------------------------------------ run to the end
    def generate(self, prompts: Sequence[Prompt], params: Union[SamplingParams, Sequence[SamplingParams], None] = None
                 ) -> List[RequestOutput]:
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        if params is None:
            params = SamplingParams()
        plist = [params] * len(prompts) if isinstance(params, SamplingParams) else list(params)
        if len(plist) != len(prompts):
            raise ConfigError("one SamplingParams per prompt, or one for all")
        was = self._no_more
        self._no_more = False
        ids = [self.submit(p, sp.max_new_tokens, sp.temperature, sp.top_p, sp.seed, sp.ignore_eos)
               for p, sp in zip(prompts, plist)]
        pending = set(ids)
        while pending:
            for r in self._step():
                pending.discard(r.request_id)
        while self._pending is not None:        # a last step may still be in flight (its tokens are dropped)
            self._step()
        self._no_more = was
        outs = []
        for rid in ids:
            r = self.requests.pop(rid)
            outs.append(RequestOutput(rid, r.prompt_ids, r.generated_ids,
                                      self._decode(r.generated_ids) if self.tokenizer is not None else None,
                                      r.finish_reason, r.preemptions))
        return outs

    # ------------------------------------------------------------------ inside
    def _step(self) -> List[Request]:
        done = self._step_ahead() if self.cfg.async_scheduling else self._step_in_turn()
        if done:
            # tokens leave the engine when a request completes: before that, make sure that no kernel gave up
            # a bounded wait on the way (it would have left part of a result unwritten)
            ops.check_kernel_status()
        return done

    def _step_in_turn(self) -> List[Request]:
        plan = self.scheduler.schedule()
        if not plan:
            return []
        logits, rows = self._launch(plan)
        if logits is None:          # every row greedy and chosen inside the head's kernel
            toks = self.sampler.tokens_from(self.runner.feedback, len(rows)).result()
        else:
            toks = self.sampler.sample(logits, *self._sampling_args(rows))
        it = iter(toks)
        sampled = [next(it) if s.samples else None for s in plan]
        self.stats["steps"] += 1
        return self.scheduler.finish_step(plan, sampled)

    def _step_ahead(self) -> List[Request]:
        """One step ahead of the device: the next batch is scheduled, built and launched while the
        tokens of the batch before are still being computed; the embedding takes them from where
        the sampling kernel left them.  The tokens are read (and requests finished) one step late."""
        plan = self.scheduler.schedule() if (self.scheduler.waiting or self.scheduler.running) else []
        launched = None
        if plan:
            logits, rows = self._launch(plan)
            if logits is None:      # every row greedy and chosen inside the head's kernel: the tokens are in feedback
                handle = self.sampler.tokens_from(self.runner.feedback, len(rows))
            else:
                handle = self.sampler.sample_async(logits, *self._sampling_args(rows), out=self.runner.feedback)
            self.scheduler.advance(plan)
            launched = (plan, handle)
            self.stats["steps"] += 1
        done: List[Request] = []
        if self._pending is not None:
            prev_plan, prev_handle = self._pending
            done = self.scheduler.resolve(prev_plan, prev_handle.result())
        self._pending = launched
        return done

    def _launch(self, plan):
        items = []
        for s in plan:
            toks = s.request.tokens(s.start, s.count)
            items.append(StepItem(s.request.slot, toks, (s.count - 1,) if s.samples else ()))
            self.stats["decode_tokens" if s.request.is_decoding else "prefill_tokens"] += s.count
        rows = [s for s in plan if s.samples]
        greedy = bool(rows) and all(r.request.temperature <= 0 for r in rows)
        logits = self.runner.step(items, greedy=greedy)
        return logits, rows

    def _sampling_args(self, rows):
        temps = [r.request.temperature for r in rows]
        if all(t <= 0 for t in temps):
            return temps, None, None                # greedy rows need neither top-p nor random numbers
        seeds = [(r.request.seed if r.request.seed is not None else self.cfg.seed) for r in rows]
        return (temps, [r.request.top_p for r in rows],
                [uniform_for(sd, r.request.request_id, len(r.request.generated_ids)) for sd, r in zip(seeds, rows)])

    def _encode(self, prompt: Prompt) -> List[int]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ConfigError("a text prompt needs a tokenizer; this model folder has none - pass token ids")
            return list(self.tokenizer.encode(prompt))
        ids = [int(t) for t in prompt]
        # negative ids have a meaning of their own inside the engine (a token still on the device): never a user's
        if ids and not 0 <= min(ids) <= max(ids) < self.model.vocab_size:
            raise ConfigError(f"prompt token ids must lie in [0, {self.model.vocab_size})")
        return ids

    def _decode(self, ids: Sequence[int]) -> str:
        return self.tokenizer.decode(list(ids))


def _maybe_tokenizer(model_dir: str):
    """The folder's tokenizer if it has one (as the reference loads it beside the weights,
    pico_vllm/run_single.py:15), else None."""
    if not any(os.path.isfile(os.path.join(model_dir, f)) for f in ("tokenizer.json", "tokenizer_config.json")):
        return None
    try:
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(model_dir)
    except Exception:
        return None
