"""The scheduler's decisions against a host-only cache manager and a fake model."""

import random

import pytest

from fastgen_b200.cache import CacheManager
from fastgen_b200.engine.scheduler import Scheduler
from fastgen_b200.parts.base import CacheSpec


def make(n_pages=16, page=8, max_batch=4, budget=32, stop=(), max_gen=None, max_length=10_000):
    spec = CacheSpec(2, 16, None)
    cache = CacheManager([spec, spec], [None, None], [None, None], page, n_pages, max_batch, max_length)
    return Scheduler(cache, max_batch, budget, stop, max_gen), cache


def fake_token(req):
    """A deterministic 'model': the next token depends on the request's tokens only."""
    return (sum(req.all_tokens()) * 31 + len(req)) % 97 + 3


def drive(sched, cache, max_steps=10_000, check=None):
    out, steps = [], 0
    while sched.has_work():
        plan = sched.plan()
        assert plan, "no progress"
        assert sum(len(e.tokens) for e in plan) <= sched.token_budget
        assert len({id(e.request) for e in plan}) == len(plan)
        for e in plan:  # what is fed is exactly the request's next tokens
            assert e.tokens == e.request.all_tokens()[e.request.fed:e.request.fed + len(e.tokens)]
            assert cache.get(id(e.request)).length == e.request.fed
        if check:
            check(plan)
        out += sched.commit(plan, [fake_token(e.request) for e in plan if e.samples])
        cache.check()
        steps += 1
        assert steps < max_steps
    return out, steps


def expected(prompt, n):
    class R:  # the same fake model, run alone
        def __init__(self): self.t = list(prompt)
        def all_tokens(self): return self.t
        def __len__(self): return len(self.t)
    r, gen = R(), []
    for _ in range(n):
        tok = fake_token(r); gen.append(tok); r.t.append(tok)
    return gen


def test_portions_follow_the_budget_and_decoders_go_first():
    sched, cache = make(n_pages=64, budget=16)
    a = sched.add("a", list(range(1, 41)), max_gen=4)
    plan = sched.plan()
    assert [len(e.tokens) for e in plan] == [16] and not plan[0].samples
    sched.commit(plan, [])
    b = sched.add("b", [5, 6, 7], max_gen=4)
    plan = sched.plan()
    # a continues its prompt, b's whole prompt fits beside it
    assert [(e.request.thread_id, len(e.tokens)) for e in plan] == [("a", 13), ("b", 3)] or \
           [(e.request.thread_id, len(e.tokens)) for e in plan] == [("a", 16)]
    sched.commit(plan, [fake_token(e.request) for e in plan if e.samples])
    while a.fed < 40:
        plan = sched.plan()
        sched.commit(plan, [fake_token(e.request) for e in plan if e.samples])
    plan = sched.plan()
    # both decode now: one token each
    assert sorted(len(e.tokens) for e in plan) == [1, 1] and all(e.samples for e in plan)


def test_outputs_equal_running_alone_under_any_interleaving():
    rng = random.Random(0)
    sched, cache = make(n_pages=40, page=8, max_batch=4, budget=24)
    prompts = {i: [rng.randrange(3, 90) for _ in range(rng.choice([1, 2, 7, 13, 30, 45]))] for i in range(12)}
    for i, p in prompts.items():
        sched.add(i, p, max_gen=rng.choice([1, 5, 16]))
    done, _ = drive(sched, cache)
    assert sorted(r.thread_id for r in done) == list(range(12))
    for r in done:
        assert r.generated == expected(prompts[r.thread_id], r.max_gen)
    assert cache.n_live == 0 and cache.free_pages() == [40]


def test_stop_token_and_length_limits():
    sched, cache = make(stop=[50], n_pages=64)
    r = sched.add("a", [1, 2, 3], max_gen=100)
    toks = iter([10, 11, 50, 12])
    while sched.has_work():
        plan = sched.plan()
        sched.commit(plan, [next(toks) for e in plan if e.samples])
    assert r.generated == [10, 11, 50]  # cut after the stop token, which is kept
    sched, cache = make(n_pages=2, page=8, max_length=16)  # the cache holds 16 tokens per request
    r = sched.add("b", list(range(1, 11)))
    done, _ = drive(sched, cache)
    assert len(r) == 16 and done == [r]


def test_request_that_can_never_fit_is_refused():
    sched, cache = make(n_pages=4, page=8)
    r = sched.add("big", list(range(40)))
    assert r.error and "never fit" in r.error and not sched.has_work()
    assert sched.take_finished() == [r]
    e = sched.add("empty", [])
    assert e.error == "empty prompt"


def test_pages_run_out_youngest_is_preempted_and_recomputed():
    # 6 pages of 8 tokens; two requests of 20 tokens each take 3 pages at admission
    sched, cache = make(n_pages=6, page=8, max_batch=4, budget=64)
    a = sched.add("a", list(range(1, 21)), max_gen=20)
    b = sched.add("b", list(range(21, 41)), max_gen=20)
    seen = []
    done, _ = drive(sched, cache, check=lambda plan: seen.append([e.request.thread_id for e in plan]))
    assert sched.n_preemptions >= 1 and b.preemptions >= 1 and a.preemptions == 0
    # the older request was never interrupted; both got exactly what they get alone
    assert a.generated == expected(list(range(1, 21)), 20)
    assert b.generated == expected(list(range(21, 41)), 20)
    assert [r.thread_id for r in done] == ["a", "b"]
    assert cache.free_pages() == [6] and cache.n_live == 0


def test_admission_is_in_order_and_waits_for_pages():
    sched, cache = make(n_pages=4, page=8, budget=64)
    a = sched.add("a", list(range(1, 25)), max_gen=2)   # 24+1 tokens -> 4 pages
    b = sched.add("b", [1, 2, 3], max_gen=2)
    plan = sched.plan()
    assert [e.request.thread_id for e in plan] == ["a"]  # b must wait although it is small
    assert [r.thread_id for r in sched.waiting] == ["b"]
    sched.commit(plan, [7])
    done, _ = drive(sched, cache)
    assert [r.thread_id for r in done] == ["a", "b"]


@pytest.mark.parametrize("seed", range(6))
def test_random_load_with_few_pages(seed):
    rng = random.Random(seed)
    sched, cache = make(n_pages=rng.choice([6, 9, 14]), page=8, max_batch=rng.choice([2, 3, 4]),
                        budget=rng.choice([8, 17, 40]))
    prompts = {}
    for i in range(15):
        prompts[i] = [rng.randrange(3, 90) for _ in range(rng.randrange(1, 30))]
        sched.add(i, prompts[i], max_gen=rng.choice([1, 3, 9, 17]))
    done, _ = drive(sched, cache)
    assert len(done) == 15
    for r in done:
        cap = min(r.max_gen, sched.capacity - len(prompts[r.thread_id]))
        assert r.generated == expected(prompts[r.thread_id], cap)
    assert cache.n_live == 0 and cache.free_pages() == [cache.groups[0].pool.n_pages]


def test_decode_runs_of_several_steps():
    """Several decode steps without looking at the tokens in between: only when every
    request decodes, nothing waits and nobody hits a limit inside the run; tokens after a
    stop token are dropped."""
    sched, cache = make(n_pages=64, page=8, budget=64, stop=[50])
    a = sched.add("a", [1, 2, 3], max_gen=20)
    b = sched.add("b", [4, 5, 6, 7], max_gen=7)
    assert sched.plan_decode_run(10) == 1          # prompts are not in yet
    plan = sched.plan()
    sched.commit(plan, [10, 20])
    assert sched.plan_decode_run(10) == 6          # b may generate 6 more
    assert cache.get(id(a)).length == 3 and len(cache.get(id(a)).pages[0]) >= 2  # pages for the run are held
    done = sched.commit_decode_run([a, b], [[11, 21], [12, 22], [50, 23], [13, 24], [14, 25], [15, 26]])
    assert a.generated == [10, 11, 12, 50] and b.generated == [20, 21, 22, 23, 24, 25, 26]
    assert {r.thread_id for r in done} == {"a", "b"} and not sched.has_work()
    cache.check()
    assert cache.free_pages() == [64]
    # a waiting request, or too few pages, mean one step at a time
    sched, cache = make(n_pages=2, page=8, budget=64)
    a = sched.add("a", list(range(1, 8)), max_gen=30)
    sched.commit(sched.plan(), [9])
    assert sched.plan_decode_run(10) == 1 or cache.free_pages() == [0]
    c = sched.add("c", [1, 2, 3], max_gen=3)
    assert sched.plan_decode_run(10) == 1


def test_min_prefill_batch_makes_short_prompts_wait_for_company():
    """The reference's rule (generate.py:600-608): while requests decode and more input may
    come, a lone newly admitted short prompt waits; it goes in with a second one, when the
    input has ended, or when nothing is decoding."""
    from fastgen_b200.cache import CacheManager
    from fastgen_b200.parts import CacheSpec

    def make():
        cache = CacheManager([CacheSpec(1, 16)], [None], [None], page_size=8, n_pages=64, max_requests=8,
                             max_length=256, dtype=None, device=None)
        return Scheduler(cache, 8, 64, (), 4, min_prefill=32, min_prefill_batch=2), cache

    def step(sched):
        plan = sched.plan()
        sched.commit(plan, [1] * sum(e.samples for e in plan))
        return plan

    sched, cache = make()
    sched.add("first", [1] * 5)           # nothing is decoding: admitted alone
    assert [e.request.thread_id for e in step(sched)] == ["first"]
    sched.add("lone", [2] * 5)            # short, alone, others decode, input open: waits
    assert [e.request.thread_id for e in step(sched)] == ["first"]
    assert len(sched.waiting) == 1 and cache.n_live == 1
    sched.add("second", [3] * 5)          # now two: both go in
    assert sorted(e.request.thread_id for e in step(sched)) == ["first", "lone", "second"]
    cache.check()

    sched, cache = make()
    sched.add("first", [1] * 5)
    step(sched)
    sched.add("long", [2] * 40)           # enough tokens by itself
    assert sorted(e.request.thread_id for e in step(sched)) == ["first", "long"]

    sched, cache = make()
    sched.add("first", [1] * 5)
    step(sched)
    sched.add("lone", [2] * 5)
    sched.input_ended = True              # no company will come
    assert sorted(e.request.thread_id for e in step(sched)) == ["first", "lone"]
    cache.check()
