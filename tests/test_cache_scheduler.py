"""The cache manager (no page lost, held twice or freed twice, under random orders of requests)
and the scheduler's decisions (admission, portions under a token budget, decoding first,
finishing, what happens when pages run out).  CPU only: the manager is built without device
tensors and the model is replaced by a stub that "samples" a fixed token."""
import random

import pytest

from pico_vllm_b200.cache import CacheManager, PagePool
from pico_vllm_b200.engine.scheduler import Request, RequestStatus, Scheduler
from pico_vllm_b200.errors import OutOfPages, PicoError, ScheduleError
from pico_vllm_b200.parts import FixedState, PagedKV

FULL = PagedKV(2, 16, None)
WIN = PagedKV(2, 16, 24)


def manager(entries=(FULL, FULL), page_size=8, num_pages=20, max_num_seqs=4, max_seq_len=160):
    return CacheManager(list(entries), page_size, num_pages, max_num_seqs, max_seq_len, allocate=False)


# ------------------------------------------------------------------ page pool
def test_pool_reuses_pages_and_refuses_double_free():
    pool = PagePool(4)
    a = pool.allocate(3)
    assert pool.available == 1 and sorted(a) == [0, 1, 2]
    with pytest.raises(OutOfPages):
        pool.allocate(2)
    assert pool.available == 1                       # all or nothing
    pool.share(a[:1])
    assert pool.release(a) == a[1:]                  # the shared page is still held once
    assert pool.release(a[:1]) == a[:1]
    with pytest.raises(PicoError):
        pool.release(a[:1])                          # freed twice
    b = pool.allocate(4)
    assert sorted(b) == [0, 1, 2, 3]                 # used again
    with pytest.raises(PicoError):
        pool.share([7])


def test_pool_hands_out_the_lowest_free_page():
    """After the whole pool has been used and given back in another order, a light load still gets the pages
    with the lowest numbers: live pages stay together instead of wandering through the pool."""
    import random
    pool = PagePool(64)
    pages = pool.allocate(64)
    random.Random(3).shuffle(pages)
    pool.release(pages)
    assert pool.allocate(5) == [0, 1, 2, 3, 4]
    pool.release([1, 3])
    assert pool.allocate(3) == [1, 3, 5]
    assert pool.available == 64 - 6


# ------------------------------------------------------------------ manager
def test_groups_by_need_and_block_tables():
    m = manager(entries=(FULL, WIN, WIN, FixedState((4,)), FULL))
    assert len(m.groups) == 2
    assert m.groups[0].entries == [0, 4] and m.groups[1].entries == [1, 2]
    assert m.entry_group[2] == (1, 1) and list(m.state_specs) == [3]
    s = m.acquire("r")
    assert m.append(s, 19) == 0                      # positions 0..18 need 3 pages of 8 in each group
    assert [g.pool.in_use for g in m.groups] == [3, 3]
    sl = m.slot_mapping(0, s, 0, 19)
    row = m.table_row(0, s)
    assert list(sl[:3]) == [row[0] * 8, row[0] * 8 + 1, row[0] * 8 + 2] and sl[8] == row[1] * 8
    m.commit(s)
    assert m.append(s, 1) == 19 and m.pages_needed(s, 5) == [1, 1]
    m.commit(s)
    m.check()
    m.release(s)
    assert [g.pool.in_use for g in m.groups] == [0, 0]
    with pytest.raises(PicoError):
        m.release(s)


def test_window_pages_come_back_when_passed():
    m = manager(entries=(FULL, WIN), num_pages=30, max_seq_len=200)
    s = m.acquire("r")
    m.append(s, 100)
    assert m.groups[1].pool.in_use == 13             # a long portion needs all its pages during the step
    m.commit(s)
    # the next query (position 100) reads keys 77..100: blocks 0..8 are dead
    assert m.groups[1].pool.in_use == 4 and m.groups[0].pool.in_use == 13
    assert m.groups[1].first_block[s] == 9 and (m.table_row(1, s)[:9] == -1).all()
    for _ in range(60):
        m.append(s, 1)
        m.commit(s)
        assert m.groups[1].pool.in_use <= 4
        m.check()
    with pytest.raises(PicoError):
        m.slot_mapping(1, s, 0, 4)                   # those positions have no page any more
    m.release(s)
    m.check()


def test_append_is_all_or_nothing_and_limits_hold():
    m = manager(num_pages=5, max_seq_len=64)
    a, b = m.acquire("a"), m.acquire("b")
    m.append(a, 30)                                  # 4 of 5 pages
    assert not m.can_append(b, 9) and m.can_append(b, 8)
    with pytest.raises(OutOfPages):
        m.append(b, 9)
    assert m.groups[0].pool.in_use == 4              # nothing was taken
    m.append(b, 8)
    with pytest.raises(ScheduleError):
        m.append(a, 40)                              # beyond the longest request the cache holds
    m.commit(a), m.commit(b)
    m.check()
    for s in range(2):
        m.acquire()
    with pytest.raises(ScheduleError):
        m.acquire()                                  # no slot left


def test_random_orders_of_requests_never_lose_a_page():
    rng = random.Random(7)
    m = manager(entries=(FULL, WIN, FULL), page_size=4, num_pages=40, max_num_seqs=6, max_seq_len=120)
    live = {}
    for it in range(3000):
        r = rng.random()
        if r < 0.15 and m.free_slots:
            live[m.acquire(it)] = 0
        elif r < 0.25 and live:
            s = rng.choice(list(live))
            m.release(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 17])
            if m.can_append(s, n):
                assert m.append(s, n) == live[s]
                if rng.random() < 0.1:
                    m.rollback(s)                    # a failed step: tokens forgotten, pages kept
                else:
                    m.commit(s)
                    live[s] += n
            else:
                with pytest.raises((OutOfPages, ScheduleError)):
                    m.append(s, n)
        if it % 50 == 0:
            m.check()
    for s in list(live):
        m.release(s)
    m.check()
    assert all(g.pool.in_use == 0 for g in m.groups)


# ------------------------------------------------------------------ scheduler
def run(sched, token=7, max_steps=10000, eos_at=None):
    """Drives the scheduler like the engine does, with the cache bookkeeping but no model."""
    log = []
    for step in range(max_steps):
        if not sched.has_work():
            break
        plan = sched.schedule()
        assert plan, "work left but nothing scheduled"
        assert sum(s.count for s in plan) <= sched.budget
        slots = [s.request.slot for s in plan]
        assert len(set(slots)) == len(slots)
        for s in plan:
            assert sched.cache.append(s.request.slot, s.count) == s.start
        for s in plan:
            sched.cache.commit(s.request.slot)
        sampled = []
        for s in plan:
            tok = None
            if s.samples:
                tok = token
                if eos_at and s.request.request_id in eos_at and len(s.request.generated_ids) + 1 == eos_at[s.request.request_id]:
                    tok = sched.eos_token_id
            sampled.append(tok)
        log.append([(s.request.request_id, s.start, s.count, s.samples) for s in plan])
        sched.finish_step(plan, sampled)
        sched.cache.check()
    assert not sched.has_work()
    return log


def req(i, n_prompt, n_new, **kw):
    return Request(i, list(range(1, n_prompt + 1)), n_new, **kw)


def test_fcfs_admission_portions_and_decode_first():
    m = manager(num_pages=100, max_num_seqs=2, max_seq_len=400)
    s = Scheduler(m, max_num_seqs=2, max_num_batched_tokens=16, prefill_chunk=10, eos_token_id=0)
    for i, (p, n) in enumerate([(25, 3), (4, 2), (6, 2)]):
        s.add(req(i, p, n))
    log = run(s)
    # step 0: request 0's first portion (10) and request 1's whole prompt (4): two running at most
    assert log[0] == [(0, 0, 10, False), (1, 0, 4, True)]
    # step 1: request 1 decodes (1 token) beside the next portion of request 0; decode tokens are
    # not crowded out by the budget
    assert log[1] == [(1, 4, 1, True), (0, 10, 10, False)]
    # request 2 is admitted only when request 1 has finished and left its slot
    first2 = next(i for i, st in enumerate(log) if any(e[0] == 2 for e in st))
    last1 = max(i for i, st in enumerate(log) if any(e[0] == 1 for e in st))
    assert first2 == last1 + 1
    # the last portion of a prompt samples the first token, then one token per step
    r0 = [e for st in log for e in st if e[0] == 0]
    assert r0 == [(0, 0, 10, False), (0, 10, 10, False), (0, 20, 5, True), (0, 25, 1, True), (0, 26, 1, True)]
    assert [r.request_id for r in s.finished] == [1, 2, 0]
    assert all(r.finish_reason == "length" and r.status is RequestStatus.FINISHED for r in s.finished)
    assert all(g.pool.in_use == 0 for g in m.groups) and m.free_slots == m.max_num_seqs


def test_eos_and_ignore_eos():
    m = manager(num_pages=50)
    s = Scheduler(m, 4, 64, eos_token_id=0)
    s.add(req(0, 5, 10))
    s.add(req(1, 5, 10, ignore_eos=True))
    run(s, eos_at={0: 3, 1: 3})
    by = {r.request_id: r for r in s.finished}
    assert by[0].finish_reason == "eos" and len(by[0].generated_ids) == 3
    assert by[1].finish_reason == "length" and len(by[1].generated_ids) == 10


def test_requests_that_can_never_fit_are_refused_at_add():
    m = manager(num_pages=4, max_seq_len=32)
    s = Scheduler(m, 4, 64)
    with pytest.raises(ScheduleError):
        s.add(req(0, 30, 3))
    with pytest.raises(ScheduleError):
        s.add(req(1, 0, 3))
    s.add(req(2, 29, 3))
    run(s)


def test_pages_run_out_the_youngest_is_preempted_and_recomputed():
    # 3 requests that each grow to 40 tokens = 5 pages, but only 11 pages: the youngest has to go
    m = manager(entries=(FULL,), num_pages=11, max_num_seqs=3, max_seq_len=88)
    s = Scheduler(m, 3, 64)
    for i in range(3):
        s.add(req(i, 20, 20))
    log = run(s)
    assert s.num_preemptions >= 1
    by = {r.request_id: r for r in s.finished}
    assert all(len(by[i].generated_ids) == 20 for i in range(3))
    assert by[0].preemptions == 0                     # the oldest always advances
    assert by[2].preemptions >= 1
    # a pre-empted request comes back as one long prompt: a portion starting at 0 longer than its prompt
    again = [e for st in log for e in st if e[0] == 2 and e[1] == 0]
    assert len(again) >= 2 and again[-1][2] > 20
    assert [g.pool.in_use for g in m.groups] == [0]


def test_a_lone_request_that_does_not_fit_raises():
    m = manager(entries=(FULL,), num_pages=3, max_seq_len=24)
    s = Scheduler(m, 2, 64)
    s.add(req(0, 20, 4))
    run(s)                                            # 24 tokens = 3 pages: fits exactly
    m2 = manager(entries=(FULL,), num_pages=3, max_seq_len=400)   # the per-request limit says yes, the pool no
    s2 = Scheduler(m2, 2, 64)
    s2.add(req(0, 20, 30))
    with pytest.raises(OutOfPages):
        run(s2)


def test_random_workloads_finish_with_every_token_and_no_page_lost():
    rng = random.Random(3)
    for trial in range(20):
        m = manager(entries=(FULL, WIN), page_size=4, num_pages=rng.choice([16, 24, 60]), max_num_seqs=rng.choice([2, 4]),
                    max_seq_len=64)
        s = Scheduler(m, m.max_num_seqs, rng.choice([8, 16, 64]), prefill_chunk=rng.choice([None, 3, 7]), eos_token_id=0)
        want = {}
        for i in range(rng.randint(3, 12)):
            p, n = rng.randint(1, 40), rng.randint(1, 20)
            s.add(req(i, p, n))
            want[i] = n
        run(s)
        assert {r.request_id: len(r.generated_ids) for r in s.finished} == want
        assert all(g.pool.in_use == 0 for g in m.groups)


def run_one_step_late(sched, rng, eos_rate=0.0, max_steps=20000):
    """Drives ``advance`` / ``resolve`` as the engine does one step ahead of the device: a step is
    scheduled and booked while the tokens of the step before are still unknown, and those are
    resolved afterwards.  A token is the end token with probability ``eos_rate``."""
    pending = None
    for _ in range(max_steps):
        if not (sched.has_work() or pending):
            break
        plan = sched.schedule() if (sched.waiting or sched.running) else []
        launched = None
        if plan:
            assert sum(s.count for s in plan) <= sched.budget
            slots = [s.request.slot for s in plan]
            assert len(set(slots)) == len(slots) and None not in slots
            for s in plan:
                assert sched.cache.append(s.request.slot, s.count) == s.start
            for s in plan:
                sched.cache.commit(s.request.slot)
            sched.advance(plan)
            launched = plan
        else:
            assert pending is not None, "nothing scheduled and nothing in flight"
        if pending is not None:
            toks = [(sched.eos_token_id if rng.random() < eos_rate else 7) for s in pending if s.samples]
            sched.resolve(pending, toks)
        pending = launched
        sched.cache.check()
    assert not sched.has_work() and pending is None


def test_random_workloads_one_step_late_with_end_tokens():
    """The workloads of the test above through ``advance`` / ``resolve``, with random end tokens: a
    request whose last token is in flight still holds its pages and slot, which must not be taken
    for "does not fit even alone"."""
    rng = random.Random(5)
    for trial in range(400):
        m = manager(entries=(FULL, WIN), page_size=4, num_pages=rng.choice([16, 24, 60]), max_num_seqs=rng.choice([2, 4]),
                    max_seq_len=64)
        s = Scheduler(m, m.max_num_seqs, rng.choice([8, 16, 64]), prefill_chunk=rng.choice([None, 3, 7]), eos_token_id=0)
        want = {}
        for i in range(rng.randint(3, 12)):
            p, n = rng.randint(1, 40), rng.randint(1, 20)
            s.add(req(i, p, n, ignore_eos=rng.random() < 0.3))
            want[i] = n
        run_one_step_late(s, rng, eos_rate=rng.choice([0.0, 0.1, 0.3]))
        got = {r.request_id: r for r in s.finished}
        assert set(got) == set(want)
        for i, r in got.items():
            assert all(t >= 0 for t in r.generated_ids)
            if r.finish_reason == "eos":
                assert r.generated_ids[-1] == 0 and 0 not in r.generated_ids[:-1] and len(r.generated_ids) <= want[i]
            else:
                assert len(r.generated_ids) == want[i]
        assert all(g.pool.in_use == 0 for g in m.groups) and m.free_slots == m.max_num_seqs
        assert not s.lingering and not s.draining


def test_a_lone_request_that_does_not_fit_still_raises_one_step_late():
    m = manager(entries=(FULL,), num_pages=3, max_seq_len=400)
    s = Scheduler(m, 2, 64)
    s.add(req(0, 20, 30))
    with pytest.raises(OutOfPages):
        run_one_step_late(s, random.Random(0))


def test_the_cache_length_guard_ends_a_request_that_add_would_have_refused():
    """``add`` refuses a request whose prompt plus ``max_new_tokens`` exceeds the longest request the cache
    holds, so a request never meets that limit on its way; the guard in ``finish_step`` / ``advance`` is for
    requests that reach the waiting line another way.  Put there directly, such a request ends with
    ``cache_length`` when it fills the cache, in turn and one step late alike."""
    for late in (False, True):
        m = manager(entries=(FULL,), num_pages=4, max_seq_len=32)
        s = Scheduler(m, 2, 64)
        r = req(0, 28, 10)
        s.waiting.append(r)                      # not through add()
        if late:
            run_one_step_late(s, random.Random(1))
        else:
            run(s)
        assert r.finish_reason == "cache_length" and r.total_len == 32
        assert all(g.pool.in_use == 0 for g in m.groups)
