"""The step function: runs a batch of (request, its next tokens) through the model, from the
cache, and returns logits at the wanted places.

``ModelRunner.step(items)`` takes pages for the new tokens, builds the index arrays on the host
(one packed int32 buffer, one host-to-device copy), calls the model once for the whole batch
and commits the tokens to the cache.  Portions of prompts and single decoded tokens share the
batch; nothing but the given tokens is computed.  Steps that hold only single tokens are
replayed from a CUDA graph per batch-size bucket (the reference captures one graph at a fixed
batch of 8 and pads with ghost rows, pico_vllm/engine.py:98-191); padding rows have position
-1, which every kernel treats as "no keys, no store".  A step that is one full portion of one
prompt (``EngineConfig.graph_prefill_tokens``) is recorded and replayed in the same way: long
prompts arrive as a row of such steps, and a replay saves the gaps between their ~250 launches.

Counterpart of the tensor building in pico_vllm/engine.py:146-181, 199-220, 325-342, which
runs one forward per prompt plus one for all decoding requests.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager
from ..config.engine import EngineConfig
from ..errors import PicoError, ScheduleError
from ..parts.base import StepShape
from .batch import Batch, GroupBatch


@dataclass
class StepItem:
    slot: int                    # the request's cache slot
    tokens: Sequence[int]        # its next tokens (one or more)
    want: Sequence[int] = ()     # places among these tokens whose logits are asked for


class _Layout:
    """Offsets of the index arrays inside one packed int32 buffer."""

    def __init__(self, T: int, S: int, R: int, n_groups: int, width: int):
        self.T, self.S, self.R, self.width = T, S, R, width
        off = 0

        def take(n):
            nonlocal off
            start = off
            off += (n + 3) // 4 * 4     # keep every array 16-byte aligned
            return start
        self.token_ids, self.positions, self.tok_seg = take(T), take(T), take(T)
        self.seg_slots, self.cu_q, self.logit_rows = take(S), take(S + 1), take(R)
        self.prefill_segs, self.decode_tokens = take(S), take(T)
        self.g_slots = [take(T) for _ in range(n_groups)]
        self.g_tables = [take(S * width) for _ in range(n_groups)]
        self.total = off


class _Staging:
    """A pinned host buffer, its device twin and an event that tells when the last copy is done
    (the host buffer is not rewritten before that)."""

    def __init__(self, n: int, device: torch.device):
        cuda = device.type == "cuda"
        self.host = torch.empty(n, dtype=torch.int32, pin_memory=cuda)
        self.dev = torch.empty(n, dtype=torch.int32, device=device)
        self.event = torch.cuda.Event() if cuda else None
        self.busy = False

    def wait(self):
        if self.event is not None and self.busy:
            self.event.synchronize()
            self.busy = False

    def upload(self, n: int):
        self.dev[:n].copy_(self.host[:n], non_blocking=True)
        if self.event is not None:
            self.event.record()
            self.busy = True


class ModelRunner:
    def __init__(self, model, cache: CacheManager, cfg: EngineConfig):
        self.model, self.cache, self.cfg = model, cache, cfg
        self.device = cache.device
        self.on_gpu = self.device.type == "cuda"
        self.views = cache.views()
        # ("decode", bucket, plans' key, greedy) or ("prefill", tokens, wanted rows, plans' key, greedy) -> recorded step
        self._graphs: dict = {}
        g = cfg.graph_prefill_tokens
        if g is None:
            g = min(cfg.prefill_chunk or cfg.max_num_batched_tokens, cfg.max_num_batched_tokens)
        self._graph_prefill_tokens = g if g > 1 else -1
        self._scratch: Optional[torch.Tensor] = None
        self._stage: Optional[_Staging] = None
        self.graph_replays = 0
        self.steps = 0
        # where the sampling kernel leaves the tokens of a step for the next step's embedding
        self.feedback = torch.zeros(max(64, cache.max_num_seqs, max(cfg.graph_batch_sizes)), dtype=torch.int32,
                                    device=self.device)
        self._num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count if self.on_gpu else 1
        # one planner per distinct plan_key() among the mixers (layers of equal sizes share a plan)
        self._planners: Dict[object, object] = {}
        for blk in model.blocks:
            mixer = getattr(blk, "mixer", None)
            if mixer is not None and hasattr(mixer, "plan") and hasattr(mixer, "plan_key"):
                self._planners.setdefault(mixer.plan_key(), mixer)

    # ------------------------------------------------------------------ buffers
    def _staging(self, n: int) -> _Staging:
        if self._stage is None or self._stage.host.numel() < n:
            if self._stage is not None:
                self._stage.wait()
            self._stage = _Staging(max(n, 4096), self.device)
        return self._stage

    def _plan(self, q_lens: List[int], starts: List[int], T: int, S: int):
        """Asks every planner for its plan of this step.  Returns (plans by plan key, a hashable key of
        all of them, float32 elements of scratch the largest of them needs)."""
        shape = StepShape(num_tokens=T, num_segments=S, q_lens=q_lens, starts=starts,
                          max_kv=max(st + n for st, n in zip(starts, q_lens)),
                          decode_only=all(n == 1 for n in q_lens), num_sms=self._num_sms, engine=self.cfg)
        plans, need = {}, 0
        for key, mixer in self._planners.items():
            plan = mixer.plan(shape)
            if plan is not None:
                plans[key] = plan
                need = max(need, int(plan.scratch_floats))
        return plans, tuple((repr(k), p.key) for k, p in plans.items()), need

    def _scratch_for(self, need: int) -> Optional[torch.Tensor]:
        """The step function's float32 scratch, grown when a plan asks for more."""
        if need <= 0:
            return None
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, dtype=torch.float32, device=self.device)
        return self._scratch

    # ------------------------------------------------------------------ the step
    def step(self, items: Sequence[StepItem], greedy: bool = False) -> Optional[torch.Tensor]:
        """Runs the items as one batch; returns float32 logits [wanted, vocab] on the device, in
        the order of the items and of each item's ``want``.  The result of a graph-replayed step
        lives in a buffer that the next such step overwrites.

        ``greedy``: the caller only wants the most likely token of every wanted row.  Where the head
        can find it inside its own kernel, the tokens are left in ``self.feedback`` (int32, one per
        wanted row, in order), no logits are written and None is returned; otherwise logits come back
        as usual and the caller chooses."""
        if not items:
            return torch.empty((0, self.model.vocab_size), dtype=torch.float32, device=self.device)
        V = self.model.vocab_size
        seen = set()
        checked = []
        for it in items:
            if len(it.tokens) < 1:
                raise PicoError("a step item needs at least one token")
            if it.slot in seen:
                raise PicoError(f"slot {it.slot} appears twice in one step")
            seen.add(it.slot)
            toks = it.tokens
            if len(toks) > 32 and not isinstance(toks, np.ndarray):
                # a portion of a prompt: one conversion serves the check here and the copy in _build
                try:
                    toks = np.asarray(toks, dtype=np.int32)
                except (OverflowError, ValueError, TypeError):
                    raise PicoError(f"token id outside [0, {V}) in a step item") from None
                it = StepItem(it.slot, toks, it.want)
            lo, hi = (int(toks.min()), int(toks.max())) if isinstance(toks, np.ndarray) else (min(toks), max(toks))
            if lo < -self.feedback.shape[0] or hi >= V:
                raise PicoError(f"token id outside [0, {V}) in a step item")
            for w in it.want:
                if not 0 <= w < len(it.tokens):
                    raise PicoError(f"wanted place {w} outside the {len(it.tokens)} tokens given")
            checked.append(it)
        items = checked
        starts = []
        done = []
        try:
            for it in items:
                starts.append(self.cache.append(it.slot, len(it.tokens)))
                done.append(it.slot)
        except Exception:
            for s in done:
                self.cache.rollback(s)
            raise
        decode_only = all(len(it.tokens) == 1 for it in items)
        try:
            if (decode_only and self.cfg.use_cuda_graph and self.on_gpu
                    and len(items) <= max(self.cfg.graph_batch_sizes)):
                logits = self._step_graph(items, starts, greedy)
            elif (len(items) == 1 and len(items[0].tokens) == self._graph_prefill_tokens and len(items[0].want) <= 1
                    and self.cfg.use_cuda_graph and self.on_gpu):
                logits = self._step_prefill_graph(items, starts, greedy)
            else:
                batch = self._build(items, starts, pad_to=None, greedy=greedy)
                logits = self.model.forward(batch, self.views)
        except Exception:
            for it in items:
                self.cache.rollback(it.slot)
            raise
        for it in items:
            self.cache.commit(it.slot)
        self.steps += 1
        return logits

    def _build(self, items: Sequence[StepItem], starts: List[int], pad_to: Optional[int],
               buffers=None, scratch=None, rows: Optional[int] = None, plans=None, greedy: bool = False) -> Batch:
        """Index arrays of the step on the device.  ``pad_to``: number of one-token segments of
        a graph bucket (the batch is padded to it and the block tables keep their full width);
        ``buffers``/``scratch``/``plans``: a recorded shape's own staging and scratch tensors, which must
        not move, and the mixers' plans it was recorded with."""
        cache = self.cache
        S_real = len(items)
        q_lens = [len(it.tokens) for it in items]
        T_real = sum(q_lens)
        S = pad_to or S_real
        T = T_real + (S - S_real)
        want_rows: List[int] = []
        at = 0
        for it, n in zip(items, q_lens):
            want_rows.extend(at + w for w in it.want)
            at += n
        R_real = len(want_rows)
        # a graph's shape is fixed: one row per segment, or the number the caller fixes
        R = R_real if pad_to is None else (S if rows is None else rows)
        if pad_to is not None and R_real > R:
            raise PicoError("more logits wanted than the graph holds")
        kv_lens = [st + n for st, n in zip(starts, q_lens)]
        if pad_to is None:
            W = min(cache.max_blocks, (-(-max(kv_lens) // cache.page_size) + 3) // 4 * 4)
        else:
            W = cache.max_blocks
        lay = _Layout(T, S, R, len(cache.groups), W)
        stage = buffers if buffers is not None else self._staging(lay.total)
        stage.wait()
        dev = stage.dev
        h = stage.host.numpy()
        tok = h[lay.token_ids:lay.token_ids + T]
        pos = h[lay.positions:lay.positions + T]
        seg = h[lay.tok_seg:lay.tok_seg + T]
        tok[:] = 0
        pos[:] = -1
        seg[:] = 0
        cu = h[lay.cu_q:lay.cu_q + S + 1]
        ss = h[lay.seg_slots:lay.seg_slots + S]
        ss[:] = 0
        single = T_real == S_real       # every segment is one token: no loop over the items
        if single:
            slot_ids = np.fromiter((it.slot for it in items), dtype=np.int64, count=S_real)
            start_pos = np.asarray(starts, dtype=np.int64)
            tok[:S_real] = np.fromiter((it.tokens[0] for it in items), dtype=np.int64, count=S_real)
            pos[:S_real] = start_pos
            seg[:] = np.arange(T, dtype=np.int32)
            cu[:] = np.arange(S + 1, dtype=np.int32)
            ss[:S_real] = slot_ids
        else:
            at = 0
            for i, (it, n, st) in enumerate(zip(items, q_lens, starts)):
                tok[at:at + n] = np.asarray(it.tokens, dtype=np.int32)
                pos[at:at + n] = np.arange(st, st + n, dtype=np.int32)
                seg[at:at + n] = i
                cu[i] = at
                ss[i] = it.slot
                at += n
            for i in range(S_real, S):      # padding segments of one token each
                seg[at] = i
                cu[i] = at
                at += 1
            cu[S] = at
        pf = [i for i, n in enumerate(q_lens) if n > 1]
        dec = [int(cu[i]) for i, n in enumerate(q_lens) if n == 1] + list(range(T_real, T))
        h[lay.prefill_segs:lay.prefill_segs + len(pf)] = np.asarray(pf, dtype=np.int32)
        h[lay.decode_tokens:lay.decode_tokens + len(dec)] = np.asarray(dec, dtype=np.int32)
        rows = h[lay.logit_rows:lay.logit_rows + R]
        rows[:] = 0
        rows[:R_real] = np.asarray(want_rows, dtype=np.int32)
        for gi, g in enumerate(cache.groups):
            sl = h[lay.g_slots[gi]:lay.g_slots[gi] + T]
            sl[:] = -1
            tb = h[lay.g_tables[gi]:lay.g_tables[gi] + S * W].reshape(S, W)
            tb[:] = 0
            if single:
                sl[:S_real] = cache.slot_mapping_single(gi, slot_ids, start_pos)
                tb[:S_real] = np.maximum(g.tables[slot_ids, :W], 0)
                continue
            at = 0
            for i, (it, n, st) in enumerate(zip(items, q_lens, starts)):
                sl[at:at + n] = cache.slot_mapping(gi, it.slot, st, n)
                row = cache.table_row(gi, it.slot)
                tb[i] = np.maximum(row[:W], 0)  # blocks without a page are never read; keep indices legal
                at += n
        stage.upload(lay.total)

        def d(off, n):
            return dev[off:off + n]
        groups = {gi: GroupBatch(d(lay.g_slots[gi], T), d(lay.g_tables[gi], S * W).view(S, W))
                  for gi in range(len(cache.groups))}
        if plans is None:
            plans, _, need = self._plan(q_lens, starts, T, S)
            scratch = self._scratch_for(need)
        return Batch(num_tokens=T, num_segments=S, token_ids=d(lay.token_ids, T), positions=d(lay.positions, T),
                     tok_seg=d(lay.tok_seg, T), seg_slots=d(lay.seg_slots, S), cu_q=d(lay.cu_q, S + 1),
                     logit_rows=d(lay.logit_rows, R), num_logit_rows=R, groups=groups, q_lens=q_lens,
                     kv_lens=kv_lens, plans=plans, scratch=scratch,
                     decode_only=all(n == 1 for n in q_lens),
                     prefill_segs=d(lay.prefill_segs, len(pf)) if len(pf) < S else None, num_prefill_segs=len(pf),
                     max_prefill_q=max([q_lens[i] for i in pf], default=0),
                     decode_tokens=d(lay.decode_tokens, len(dec)) if len(dec) < T else None,
                     num_decode_tokens=len(dec), feedback=self.feedback,
                     greedy_out=self.feedback if greedy and R > 0 else None)

    # ------------------------------------------------------------------ CUDA graph replay of decode steps
    def _bucket(self, n: int) -> int:
        return min(b for b in self.cfg.graph_batch_sizes if b >= n)

    def _step_graph(self, items: Sequence[StepItem], starts: List[int], greedy: bool = False) -> Optional[torch.Tensor]:
        B = self._bucket(len(items))
        # every segment has one token; logits (or greedy tokens) are computed for every row of the bucket
        full = [StepItem(it.slot, it.tokens, (0,)) for it in items]
        rows = [i for i, it in enumerate(items) if len(it.want)]
        greedy = greedy and len(rows) == len(items)        # tokens land in row order: only when every row is wanted
        # a recorded step holds for one set of plans: as contexts grow a bucket may be recorded a few times
        # (for attention: once per number of splits of the key range)
        plans, plan_key, need = self._plan([1] * len(items), starts, B, B)
        key = ("decode", B, plan_key, greedy)
        entry = self._graphs.get(key)
        if entry is None:
            logits = self._record(key, full, starts, B, B, plans, need, greedy)
        else:
            self._build(full, starts, pad_to=B, buffers=entry["buffers"], scratch=entry["scratch"], plans=entry["plans"],
                        greedy=greedy)
            entry["graph"].replay()
            ops._count(entry["launches"])
            logits = entry["logits"]
        self.graph_replays += 1
        if logits is None:
            return None
        if len(rows) == len(items):
            return logits[:len(items)]
        return logits[torch.tensor(rows, dtype=torch.long, device=self.device)] if rows else logits[:0]

    def _step_prefill_graph(self, items: Sequence[StepItem], starts: List[int], greedy: bool = False) -> Optional[torch.Tensor]:
        """One full portion of one prompt: the same work every time but for the index arrays, so it is
        recorded once (per number of wanted rows, 0 or 1, and per set of plans) and replayed over its own
        staging buffers."""
        T, R = len(items[0].tokens), len(items[0].want)
        greedy = greedy and R == 1
        plans, plan_key, need = self._plan([T], starts, T, 1)
        key = ("prefill", T, R, plan_key, greedy)
        entry = self._graphs.get(key)
        if entry is None:
            logits = self._record(key, items, starts, 1, R, plans, need, greedy)
        else:
            self._build(items, starts, pad_to=1, buffers=entry["buffers"], scratch=entry["scratch"], rows=R,
                        plans=entry["plans"], greedy=greedy)
            entry["graph"].replay()
            ops._count(entry["launches"])
            logits = entry["logits"]
        self.graph_replays += 1
        return logits

    def _record(self, key, items: Sequence[StepItem], starts: List[int], S: int, R: int, plans, need: int,
                greedy: bool = False) -> Optional[torch.Tensor]:
        """First step of a shape: a graph keeps the addresses it was recorded with, so the shape owns its
        staging buffer and its scratch."""
        T = sum(len(it.tokens) for it in items) + (S - len(items))
        lay = _Layout(T, S, R, len(self.cache.groups), self.cache.max_blocks)
        buffers = _Staging(lay.total, self.device)
        scratch = torch.empty(need, dtype=torch.float32, device=self.device) if need > 0 else None
        batch = self._build(items, starts, pad_to=S, buffers=buffers, scratch=scratch, rows=R, plans=plans, greedy=greedy)
        return self._run_and_record(key, batch, {"buffers": buffers, "scratch": scratch, "plans": plans})

    def _run_and_record(self, key, batch: Batch, entry: dict) -> torch.Tensor:
        """The first step of a shape: runs it once, directly (this is the step itself, and it warms up the
        libraries), then records the same work into a graph over the same buffers.  Recording executes
        nothing and the recorded graph is not replayed here: the step's work happens exactly once, so a
        mixer that advances per-request state of its own is stepped once, like the cache.  Returns
        the direct run's logits."""
        logits = self.model.forward(batch, self.views)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        before = ops.launches
        with torch.cuda.graph(graph):
            recorded = self.model.forward(batch, self.views)
        entry.update(graph=graph, logits=recorded, launches=ops.launches - before, batch=batch)
        self._graphs[key] = entry
        return logits
