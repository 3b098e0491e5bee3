"""Continuous-batching scheduler: admits requests first come first served, cuts prompts into
portions under a token budget, decodes, finishes and frees.

The reference keeps four lists (waiting / prefilling / decoding / finished), admits up to
``max_num_seqs`` = 4 requests, runs each new prompt whole in a forward of its own and has no
token budget, no portions and no page check (pico_vllm/scheduler.py:66-180; chunked prefill
is on its to-do list, TODO.md:3).  Here one step holds single tokens of decoding requests
first, then portions of prompts, oldest request first, up to ``max_num_batched_tokens``; a
prompt may span many steps and the request turns decoding in the step that runs its last
portion, which also yields its first token.

When pages run out: the youngest running request is pre-empted - its pages and slot are given
back and it returns to the front of the waiting line with everything it has generated so far,
to be recomputed as one long prompt later.  The oldest request therefore always advances.  A
request that cannot fit even alone raises OutOfPages when it is scheduled; one whose prompt
plus ``max_new_tokens`` exceeds the longest request the cache can hold is refused at ``add``.
The reference raises from the allocator instead (pico_vllm/blockmanager.py:77-78).

States: WAITING -> RUNNING -> FINISHED, and RUNNING -> WAITING again through pre-emption
(the reference: WAITING -> PREFILL -> DECODING -> FINISHED -> CLOSED, pico_vllm/scheduler.py:7-12).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Deque, List, Optional, Sequence, Tuple

from ..errors import OutOfPages, ScheduleError


class RequestStatus(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class Request:
    request_id: int
    prompt_ids: List[int]
    max_new_tokens: int
    temperature: float = 0.0
    top_p: float = 1.0
    ignore_eos: bool = False
    seed: Optional[int] = None
    generated_ids: List[int] = field(default_factory=list)
    status: RequestStatus = RequestStatus.WAITING
    slot: Optional[int] = None
    num_computed: int = 0          # tokens of prompt + generated that are in the cache
    preemptions: int = 0
    finish_reason: Optional[str] = None
    in_flight: int = 0             # launched steps of this request whose tokens the host has not read yet

    @property
    def all_ids(self) -> List[int]:
        return self.prompt_ids + self.generated_ids

    @property
    def total_len(self) -> int:
        return len(self.prompt_ids) + len(self.generated_ids)

    def tokens(self, start: int, count: int) -> List[int]:
        """Tokens start .. start+count-1 of prompt + generated, without joining the two lists."""
        n = len(self.prompt_ids)
        if start >= n:
            return self.generated_ids[start - n:start - n + count]
        if start + count <= n:
            return self.prompt_ids[start:start + count]
        return self.prompt_ids[start:] + self.generated_ids[:start + count - n]

    @property
    def remaining(self) -> int:
        """Tokens that still have to go through the model before the next one can be sampled."""
        return self.total_len - self.num_computed

    @property
    def is_decoding(self) -> bool:
        return self.remaining == 1 and len(self.generated_ids) > 0


@dataclass
class Scheduled:
    request: Request
    start: int                     # index into request.all_ids of the first token of this portion
    count: int                     # tokens of this portion
    samples: bool                  # the portion reaches the end: its last logits yield a token


class Scheduler:
    def __init__(self, cache, max_num_seqs: int, max_num_batched_tokens: int,
                 prefill_chunk: Optional[int] = None, eos_token_id: Optional[int] = None):
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.budget = max_num_batched_tokens
        self.chunk = prefill_chunk or max_num_batched_tokens
        self.eos_token_id = eos_token_id
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []       # in order of admission: oldest first
        self.finished: List[Request] = []
        self.draining: List[Request] = []      # their last token is being computed; not scheduled again
        self.lingering: List[Request] = []     # ended by their end token while a later step of theirs was in flight
        self.num_preemptions = 0

    # ------------------------------------------------------------------ requests in and out
    def add(self, request: Request) -> None:
        if not request.prompt_ids:
            raise ScheduleError("a request needs at least one prompt token")
        if request.max_new_tokens < 1:
            raise ScheduleError("max_new_tokens must be at least 1")
        longest = len(request.prompt_ids) + request.max_new_tokens
        if longest > self.cache.max_seq_len:
            raise ScheduleError(f"prompt ({len(request.prompt_ids)}) + max_new_tokens ({request.max_new_tokens}) "
                                f"exceeds the longest request the cache holds ({self.cache.max_seq_len})")
        request.status = RequestStatus.WAITING
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self.draining)

    def _held_in_flight(self) -> bool:
        """True while requests that will not be scheduled again still hold pages or a slot, because a
        launched step of theirs has not been read yet (one step ahead of the device): what they hold
        comes back at the next ``resolve``, so "the cache to itself" cannot be judged before that."""
        return any(r.slot is not None for r in self.draining) or any(r.slot is not None for r in self.lingering)

    def _preempt(self, request: Request) -> None:
        self.cache.release(request.slot)
        request.slot = None
        request.num_computed = 0
        request.status = RequestStatus.WAITING
        request.preemptions += 1
        self.num_preemptions += 1
        self.running.remove(request)
        self.waiting.appendleft(request)

    # ------------------------------------------------------------------ one step's plan
    def schedule(self) -> List[Scheduled]:
        budget = self.budget
        plan: List[Scheduled] = []
        reserve = [0] * len(self.cache.groups)
        preempted: set = set()

        def fits(req: Request, n: int) -> bool:
            return self.cache.can_append(req.slot, n, reserve)

        def take(req: Request, n: int) -> None:
            nonlocal budget
            need = self.cache.pages_needed(req.slot, n)
            for i, p in enumerate(need):
                reserve[i] += p
            plan.append(Scheduled(req, req.num_computed, n, req.num_computed + n == req.total_len))
            budget -= n


        # 1. running requests: one token for each decoding request first, then portions of
        #    prompts, oldest request first in both passes
        for req in ([r for r in self.running if r.is_decoding] + [r for r in self.running if not r.is_decoding]):
            if req.status is not RequestStatus.RUNNING:
                continue                # pre-empted earlier in this step
            if budget <= 0:
                break
            n = 1 if req.is_decoding else min(req.remaining, self.chunk, budget)
            gone = False
            while not fits(req, n):
                victim = self.running[-1]
                if victim is req:
                    if len(self.running) == 1 and not plan:
                        # alone and still too big: a shorter portion may fit
                        while n > 1 and not fits(req, n):
                            n -= 1
                        if fits(req, n):
                            break
                        if self._held_in_flight():
                            return plan         # empty: the caller reads the step in flight, then asks again
                        raise OutOfPages(f"request {req.request_id} cannot go on even with the cache to itself "
                                         f"({req.total_len} tokens; {self.cache.num_pages} pages of "
                                         f"{self.cache.page_size})")
                    self._preempt(req)
                    preempted.add(req.request_id)
                    gone = True
                    break
                # the victim may already be in this step's plan: take it out again
                for k, sch in enumerate(plan):
                    if sch.request is victim:
                        need = self.cache.pages_needed(victim.slot, sch.count)
                        for gi, p in enumerate(need):
                            reserve[gi] -= p
                        budget += sch.count
                        del plan[k]
                        break
                self._preempt(victim)
                preempted.add(victim.request_id)
            if not gone:
                take(req, n)

        # 2. new requests, first come first served, while slots, budget and pages last
        while (self.waiting and budget > 0 and len(self.running) < self.max_num_seqs
               and self.cache.free_slots > 0):
            req = self.waiting[0]
            if req.request_id in preempted:
                break                   # just pre-empted for lack of pages: not in the same step
            slot = self.cache.acquire(req)
            req.slot = slot
            n = min(req.remaining, self.chunk, budget)
            if not fits(req, n):
                while n > 1 and not fits(req, n):
                    n -= 1
                if not fits(req, n) or (self.running and n < min(req.remaining, self.chunk, budget)):
                    # not enough pages now; wait for running requests to finish
                    self.cache.release(slot)
                    req.slot = None
                    if not self.running and not plan and not self._held_in_flight():
                        raise OutOfPages(f"request {req.request_id} does not fit the cache even alone")
                    break
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            take(req, n)
        return plan

    # ------------------------------------------------------------------ one step ahead
    # The engine may launch step k+1 before it has read the tokens of step k.  ``advance`` books a
    # launched step without the token values (a placeholder stands for each token to come: -(j+1)
    # for the j-th sampled row, which is what the next step's embedding reads on the device);
    # ``resolve`` puts the values in when they arrive and finishes requests.  A request that ends by
    # its token count is known at ``advance`` and is not scheduled again; one that ends by its end
    # token has by then been launched once more: that work is thrown away, and its pages and slot are
    # given back only when ``resolve`` is called for that later step (until then it is in ``lingering``).  While
    # such a request, or one in ``draining``, still holds pages, ``schedule`` does not judge that a request "does
    # not fit even alone": it returns what it has (maybe nothing) and the caller asks again after ``resolve``.
    def advance(self, plan: Sequence[Scheduled]) -> None:
        j = 0
        for s in plan:
            req = s.request
            req.num_computed += s.count
            if not s.samples:
                continue
            req.generated_ids.append(-(j + 1))
            j += 1
            req.in_flight += 1
            if len(req.generated_ids) >= req.max_new_tokens or req.total_len >= self.cache.max_seq_len:
                # the last token is on its way: nothing more to compute for this request
                req.finish_reason = "length" if len(req.generated_ids) >= req.max_new_tokens else "cache_length"
                if req in self.running:
                    self.running.remove(req)
                    self.draining.append(req)

    def resolve(self, plan: Sequence[Scheduled], tokens: Sequence[int]) -> List[Request]:
        """Token values of a step booked with ``advance``.  Returns the requests that finished."""
        done: List[Request] = []
        it = iter(tokens)
        for j, s in enumerate(p for p in plan if p.samples):
            req, tok = s.request, int(next(it))
            req.in_flight -= 1
            if req.status is RequestStatus.FINISHED:
                # ended by its end token one step earlier; this step's token is dropped
                if req.in_flight == 0 and req.slot is not None:
                    self.cache.release(req.slot)
                    req.slot = None
                    self.lingering.remove(req)
                continue
            # the oldest placeholder of this request is this step's token
            at = next(i for i, t in enumerate(req.generated_ids) if t < 0)
            req.generated_ids[at] = tok
            hit_eos = not req.ignore_eos and self.eos_token_id is not None and tok == self.eos_token_id
            last = at == len(req.generated_ids) - 1
            if hit_eos or (last and req in self.draining):
                if hit_eos:
                    req.finish_reason = "eos"
                    del req.generated_ids[at + 1:]      # placeholders of steps launched after the end token
                    req.num_computed = min(req.num_computed, req.total_len)
                req.status = RequestStatus.FINISHED
                if req in self.running:
                    self.running.remove(req)
                if req in self.draining:
                    self.draining.remove(req)
                if req in self.waiting:
                    self.waiting.remove(req)
                if req.in_flight == 0 and req.slot is not None:
                    self.cache.release(req.slot)
                    req.slot = None
                elif req.slot is not None:
                    self.lingering.append(req)
                self.finished.append(req)
                done.append(req)
        return done

    # ------------------------------------------------------------------ after the step
    def finish_step(self, plan: Sequence[Scheduled], sampled: Sequence[Optional[int]]) -> List[Request]:
        """``sampled[i]`` is the token chosen for ``plan[i]`` (None where nothing was sampled).
        Returns the requests that finished; their pages and slots are already given back."""
        done: List[Request] = []
        for s, tok in zip(plan, sampled):
            req = s.request
            req.num_computed += s.count
            if not s.samples:
                continue
            if tok is None:
                raise ScheduleError(f"request {req.request_id} reached its end but no token was sampled")
            req.generated_ids.append(int(tok))
            reason = None
            if not req.ignore_eos and self.eos_token_id is not None and int(tok) == self.eos_token_id:
                reason = "eos"
            elif len(req.generated_ids) >= req.max_new_tokens:
                reason = "length"
            elif req.total_len >= self.cache.max_seq_len:
                reason = "cache_length"
            if reason:
                req.finish_reason = reason
                req.status = RequestStatus.FINISHED
                self.cache.release(req.slot)
                req.slot = None
                self.running.remove(req)
                self.finished.append(req)
                done.append(req)
        return done
