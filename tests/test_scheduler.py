"""The scheduler's decisions on the host (no GPU): admission order and caps, worst-case
reservation, portions under a token budget, decode before prompts, finishing frees, and what
happens when pages run out (the newest running request is preempted and recomputed).  The
cases of the reference's tests/test_scheduler.py are kept in this engine's terms."""

from __future__ import annotations

import pytest

from nanospec_b200.cache import CacheManager
from nanospec_b200.engine.scheduler import Request, RequestTooLarge, SamplingParams, Scheduler
from nanospec_b200.parts import CacheNeed


def cache(num_blocks=64, block_size=4, slots=16, window=0):
    return CacheManager([(CacheNeed(1, 8, window), None)], num_blocks, block_size, slots)


def req(i, n, max_tokens=4):
    return Request(i, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, seed=i))


def run_step(s: Scheduler, next_token=lambda r: 7):
    """What the engine does around a step, without a model: reserve, commit, emit, finish."""
    batch = s.next_batch()
    for sch in batch:
        s.cache.extend(sch.req.id, len(sch.tokens))
    for sch in batch:
        s.cache.trim(sch.req.id)
        sch.req.committed += len(sch.tokens)
        if sch.samples:
            sch.req.out_tokens.append(next_token(sch.req))
            if len(sch.req.out_tokens) >= sch.req.params.max_tokens:
                s.finish(sch.req)
    s.cache.check()
    return batch


def test_staggered_admission_and_decode_order():
    s = Scheduler(cache(), max_admit=1)
    for i in range(3):
        s.add(req(i, 5))
    assert [(x.req.id, len(x.tokens), x.samples) for x in run_step(s)] == [(0, 5, True)]
    assert [(x.req.id, len(x.tokens)) for x in run_step(s)] == [(0, 1), (1, 5)]
    assert [(x.req.id, len(x.tokens)) for x in run_step(s)] == [(0, 1), (1, 1), (2, 5)]
    s.max_running = 3
    s.add(req(3, 5))
    assert 3 not in [x.req.id for x in run_step(s)]  # concurrency cap
    assert [r.id for r in s.waiting] == [3]


def test_admission_waits_for_pages_and_finish_frees():
    c = cache(num_blocks=4, block_size=4)
    s = Scheduler(c, max_admit=8)
    s.add(req(0, 12))  # 12 + 4 - 1 positions -> 4 pages
    s.add(req(1, 6))   # 3 pages: does not fit beside request 0
    s.add(req(2, 2))   # 2 pages: would fit now, but admission is first-in first-out: it stays behind request 1
    assert [x.req.id for x in s.next_batch()] == [0]
    assert [r.id for r in s.waiting] == [1, 2]
    s.finish(s.running[0])
    assert c.free_pages() == [4]
    assert [x.req.id for x in s.next_batch()] == [1]  # 3 reserved, one page of headroom left
    s.finish(s.running[0])
    assert [x.req.id for x in s.next_batch()] == [2]
    for r in list(s.running):
        s.finish(r)
    assert not s.has_work and c.free_pages() == [4]
    c.check()


def test_reservation_means_growth_never_fails():
    c = cache(num_blocks=12, block_size=4)
    s = Scheduler(c, max_admit=8)
    for i in range(6):
        s.add(req(i, 6, max_tokens=11))  # 16 positions -> 4 pages each: three fit at a time
    done = 0
    for _ in range(200):
        if not s.has_work:
            break
        before = {r.id for r in s.running}
        run_step(s)
        assert len(s.running) <= 3
        done += len(before - {r.id for r in s.running})
    assert not s.has_work and s.preempted_total == 0 and c.free_pages() == [12]


def test_a_request_that_can_never_fit_is_refused_when_added():
    s = Scheduler(cache(num_blocks=4, block_size=4))
    with pytest.raises(RequestTooLarge):
        s.add(req(0, 14, max_tokens=4))  # 17 positions -> 5 pages
    s.add(req(1, 13, max_tokens=4))      # 16 positions fit exactly


def test_prompts_are_cut_into_portions_under_the_budget():
    s = Scheduler(cache(num_blocks=64), max_admit=4, max_step_tokens=10, prefill_chunk=6)
    s.add(req(0, 15))
    s.add(req(1, 3))
    b = run_step(s)
    assert [(x.req.id, len(x.tokens), x.samples) for x in b] == [(0, 6, False), (1, 3, True)]
    b = run_step(s)  # the decoding request first, then the next portion of the prompt
    assert [(x.req.id, len(x.tokens), x.samples) for x in b] == [(1, 1, True), (0, 6, False)]
    b = run_step(s)
    assert [(x.req.id, len(x.tokens), x.samples) for x in b] == [(1, 1, True), (0, 3, True)]
    assert b[1].tokens == [13, 14, 15]
    b = run_step(s)
    assert [(x.req.id, len(x.tokens)) for x in b] == [(0, 1), (1, 1)]  # both decode now: oldest first
    assert b[0].tokens == [7]  # the token sampled after the last portion


def test_budget_smaller_than_the_decoders_leaves_some_out():
    s = Scheduler(cache(), max_admit=8, max_step_tokens=2)
    for i in range(3):
        s.add(req(i, 1, max_tokens=8))
    assert len(run_step(s)) == 2
    ids = [x.req.id for x in run_step(s)]
    assert len(ids) == 2 and ids == [0, 1]  # oldest first; request 2 waits for budget


def test_optimistic_admission_preempts_the_newest_and_recomputes_it():
    c = cache(num_blocks=6, block_size=4)
    s = Scheduler(c, max_admit=8, admission="optimistic")
    s.add(req(0, 8, max_tokens=12))   # needs 5 pages in the end
    s.add(req(1, 8, max_tokens=12))
    tokens = {0: iter(range(100, 200)), 1: iter(range(200, 300))}
    run_step(s, lambda r: next(tokens[r.id]))
    assert [r.id for r in s.running] == [0, 1] and c.free_pages() == [2]
    for _ in range(4):
        run_step(s, lambda r: next(tokens[r.id]))
    assert c.free_pages() == [0] and s.preempted_total == 0
    b = run_step(s, lambda r: next(tokens[r.id]))  # both need a fourth page and none is free
    assert s.preempted_total == 1
    r1 = s.waiting[0]
    assert r1.id == 1 and r1.state == "waiting" and r1.committed == 0 and r1.preemptions == 1
    assert r1.out_tokens == list(range(200, 205))  # what it had emitted is kept
    assert [x.req.id for x in b] == [0]
    # the older request runs to its end, then the preempted one is recomputed from prompt + output
    while s.running and s.running[0].id == 0:
        b = run_step(s, lambda r: next(tokens[r.id]))
    b = run_step(s, lambda r: next(tokens[r.id])) if not any(x.req.id == 1 for x in b) else b
    first = [x for x in b if x.req.id == 1][0]
    assert first.tokens[:8] == list(range(1, 9)) and first.tokens[8:] == list(range(200, 200 + len(first.tokens) - 8))
    while s.has_work:
        run_step(s, lambda r: next(tokens[r.id]))
    assert c.free_pages() == [6]
    assert len(r1.out_tokens) == 12 and r1.out_tokens[:5] == list(range(200, 205))


def test_optimistic_mode_never_deadlocks_under_pressure():
    c = cache(num_blocks=10, block_size=4, slots=8)
    s = Scheduler(c, max_admit=4, admission="optimistic", max_step_tokens=16, prefill_chunk=8)
    reqs = [req(i, 5 + 3 * i, max_tokens=10) for i in range(7)]
    for r in reqs:
        s.add(r)
    steps = 0
    while s.has_work:
        run_step(s)
        steps += 1
        assert steps < 2000
    assert all(len(r.out_tokens) == 10 and r.state == "done" for r in reqs)
    assert s.preempted_total > 0 and c.free_pages() == [10]


def test_restart_requeues_at_the_front():
    s = Scheduler(cache(), max_admit=8)
    s.add(req(0, 4)), s.add(req(1, 4)), s.add(req(2, 4))
    s.max_admit = 2
    run_step(s)
    s.restart(s.running[1])
    assert [r.id for r in s.waiting] == [1, 2] and s.waiting[0].committed == 0 and s.waiting[0].out_tokens == [7]


def test_windowed_groups_reserve_their_peak_only():
    c = cache(num_blocks=6, block_size=4, window=6)
    s = Scheduler(c, max_admit=8, prefill_chunk=4, max_step_tokens=8)
    s.add(req(0, 20, max_tokens=30))  # 49 positions would need 13 pages without the window; the peak is 4
    s.add(req(1, 2, max_tokens=3))
    steps = 0
    while s.has_work:
        run_step(s)
        steps += 1
        assert steps < 200
    assert c.free_pages() == [6]


@pytest.mark.parametrize("admission", ["reserve", "optimistic"])
def test_could_admit_says_what_next_batch_does(admission):
    """The engine launches a step ahead of its predecessor's results only while `could_admit` is false: it
    must not be false when the next batch would take the head of the queue."""
    import random

    rng = random.Random(5)
    for trial in range(30):
        c = cache(num_blocks=rng.choice([6, 10, 24]), block_size=4, slots=rng.choice([2, 3, 8]))
        s = Scheduler(c, max_admit=rng.choice([1, 4]), max_running=rng.choice([None, 2, 3]), max_step_tokens=64,
                      prefill_chunk=rng.choice([4, 16]), admission=admission)
        next_id = 0
        for step in range(40):
            if rng.random() < 0.5:
                n, mt = rng.randrange(1, 12), rng.randrange(1, 6)
                if c.groups[0].blocks_for(n + mt - 1) <= c.num_blocks:
                    s.add(req(next_id, n, mt))
                    next_id += 1
            said = s.could_admit()
            before, preempted = len(s.running), s.preempted_total
            run = [r.id for r in s.running]
            batch = s.next_batch()
            took = any(x.req.id not in run for x in batch)
            # never "no" where the batch then takes somebody: a launch ahead must not pass over an admission that
            # was possible.  Under reservation the answer is exact; the optimistic rule also counts the pages that
            # the running requests take in the same step, so there a "yes" may still be followed by no admission.
            assert said or not took, (trial, step, [r.id for r in s.waiting], run)
            if admission == "reserve" and s.preempted_total == preempted:
                assert said == took, (trial, step, said, [r.id for r in s.waiting], run)
            for sch in batch:
                s.cache.extend(sch.req.id, len(sch.tokens))
            for sch in batch:
                s.cache.trim(sch.req.id)
                sch.req.committed += len(sch.tokens)
                if sch.samples:
                    sch.req.out_tokens.append(7)
                    if len(sch.req.out_tokens) >= sch.req.params.max_tokens:
                        s.finish(sch.req)
            s.cache.check()


def test_a_requests_uniforms_are_the_stream_of_single_draws():
    import torch

    from nanospec_b200.engine import Request, SamplingParams

    r = Request(0, [1], SamplingParams(seed=5))
    g = torch.Generator().manual_seed(5)
    assert [r.next_uniform() for _ in range(21)] == [float(torch.rand(1, generator=g)) for _ in range(21)]


def test_a_batch_composed_while_a_step_is_in_flight_admits_and_takes_tokens_on_the_device():
    """`next_batch(ahead=...)`: the requests whose next token the step in flight samples bring a placeholder with
    the row to take it from, unless that token is their last; a waiting request that fits is admitted beside them;
    a portion of a prompt goes on from where the step in flight leaves it.  Optimistic admission declines."""
    s = Scheduler(cache(), max_admit=1, prefill_chunk=6)
    a, b, c = req(0, 5, max_tokens=3), req(1, 9, max_tokens=4), req(2, 4, max_tokens=2)
    for r in (a, b, c):
        s.add(r)
    run_step(s)                                        # a's prompt; a has one token now
    first = s.next_batch()                             # a decodes, b's first portion
    assert [(x.req.id, len(x.tokens), x.samples) for x in first] == [(0, 1, True), (1, 6, False)]
    for sch in first:                                  # the step is launched: pages taken, positions committed, no token yet
        s.cache.extend(sch.req.id, len(sch.tokens))
        sch.req.committed += len(sch.tokens)
    ahead = s.next_batch(ahead={id(a): 0})
    assert [(x.req.id, len(x.tokens), x.samples, x.from_row) for x in ahead] == [(0, 1, True, 0), (1, 3, True, None), (2, 4, True, None)]
    assert ahead[0].tokens == [0] and ahead[1].tokens == [7, 8, 9] and c.state == "running"
    for sch in ahead:
        s.cache.extend(sch.req.id, len(sch.tokens))
        sch.req.committed += len(sch.tokens)
    a.out_tokens.append(7)                             # the first step's token arrives: a has two of its three ...
    # ... and the step in flight samples its last: the batch after it has no row for a; b and c, whose first tokens
    # are in flight, go on with placeholders
    after = s.next_batch(ahead={id(a): 0, id(b): 1, id(c): 2})
    assert [(x.req.id, x.tokens, x.from_row) for x in after] == [(1, [0], 1), (2, [0], 2)]
    s.cache.check()
    assert Scheduler(cache(), admission="optimistic").next_batch(ahead={}) is None
