"""The scheduler's decisions, on the host, with a stand-in for the model: admission, the token budget,
chunked prefill, decoding, finishing, and what happens when pages run out."""
import pytest

from tensorline_b200.cache import CacheManager, PagedKV
from tensorline_b200.engine.scheduler import Plan, Request, RequestDoesNotFit, Scheduler, Slice
from tensorline_b200.sampling import SamplingParams


def make(pages=16, page=4, seqs=4, budget=8, max_len=64, sharing=False, window=None, **kw):
    cache = CacheManager({0: PagedKV(1, 16, window)}, page_size=page, num_pages=pages, max_num_seqs=seqs,
                         max_model_len=max_len, prefix_caching=sharing)
    return Scheduler(cache, max_num_seqs=seqs, max_batched_tokens=budget, max_model_len=max_len, **kw), cache


def shape(plan):
    return [(s.request.rid, s.count) for s in plan]


def req(rid, n, max_tokens=4, first=0):
    return Request(rid, n, list(range(first, first + n)), SamplingParams(max_tokens=max_tokens), set())


def run(s, token=lambda r: 1000 + r.num_generated, limit=500):
    """Drive the scheduler to the end, 'sampling' `token(request)`; returns the list of plans."""
    plans = []
    for _ in range(limit):
        if not s.has_work():
            return plans
        plan = s.schedule()
        plans.append(shape(plan))
        done_prefill = [sl.request for sl in plan if sl.wants_logits]
        s.computed(plan)
        for r in done_prefill:
            s.accept(r, token(r))
        s.cache.check()
    raise AssertionError("the scheduler did not finish")


def test_budget_cuts_prompts_into_portions_and_decodes_beside_them():
    s, cache = make(budget=8)
    a, b = req(0, 13), req(1, 5)
    s.add(a); s.add(b)
    assert shape(s.schedule()) == [(0, 8)]           # b waits: the budget is spent
    s.computed([Slice(a, 0, 8)])
    plan = s.schedule()
    assert shape(plan) == [(0, 5), (1, 3)]           # rest of a, then what is left for b
    s.computed(plan)
    s.accept(a, 7)
    plan = s.schedule()
    assert shape(plan) == [(0, 1), (1, 2)]           # a decodes beside b's portion
    assert s.max_running_seen == 2


def test_finishing_reasons_and_pages_come_back():
    s, cache = make()
    a = req(0, 3, max_tokens=2)
    b = Request(1, 3, [5, 6, 7], SamplingParams(max_tokens=10), {42})
    s.add(a); s.add(b)
    run(s, token=lambda r: 42 if r.rid == 1 and r.num_generated == 1 else 9)
    assert a.stats.finish_reason == "length" and a.output_tokens == [9, 9]
    assert b.stats.finish_reason == "stop" and b.output_tokens == [9]  # the stop token is not kept
    assert cache.num_free_pages() == cache.num_pages and cache.num_free_slots == 4
    assert s.finished == {"length": 1, "stop": 1}


def test_max_model_len_ends_a_request_and_long_prompts_are_refused():
    s, _ = make(max_len=8)
    a = req(0, 6, max_tokens=100)
    s.add(a)
    run(s)
    assert a.stats.finish_reason == "length" and len(a.tokens) == 8
    with pytest.raises(ValueError, match="max_model_len"):
        s.add(req(1, 8))


def test_sequence_limit_queues_requests():
    s, _ = make(seqs=2, budget=64)
    rs = [req(i, 3, max_tokens=3) for i in range(5)]
    for r in rs:
        s.add(r)
    plans = run(s)
    assert max(len(p) for p in plans) == 2 and all(r.done and r.num_generated == 3 for r in rs)


def test_pages_run_out_newest_is_preempted_and_recomputed():
    """4 pages of 4 tokens; two requests of 6 tokens each grow until the pool is full: the newest is
    preempted, gives everything back, waits at the front and is recomputed with its generated tokens."""
    s, cache = make(pages=4, page=4, budget=64)
    a, b = req(0, 6, max_tokens=6), req(1, 6, max_tokens=6, first=50)
    s.add(a); s.add(b)
    plans = run(s)
    assert s.preemptions >= 1
    assert a.num_generated == 6 and b.num_generated == 6
    recomputed = [p for p in plans if any(rid == 1 and n > 6 for rid, n in p)]
    assert recomputed, "the preempted request must come back with prompt and generated tokens as one portion"
    assert cache.num_free_pages() == 4
    first_preempt = next(i for i, p in enumerate(plans) if (1, 1) not in p and i > 0 and (0, 1) in p)
    assert all(rid != 1 for rid, _ in plans[first_preempt])            # the victim is out of that step's plan


def test_request_that_can_never_fit_fails_instead_of_hanging():
    s, cache = make(pages=2, page=4, budget=64)
    big = req(0, 9)                                                    # needs 3 pages, the pool has 2
    s.add(big)
    plan = s.schedule()
    assert not plan and plan.failed == [big] and s.failed == [big]
    assert isinstance(big.error, RequestDoesNotFit) and big.done and not s.has_work()
    grows = req(1, 7, max_tokens=5)                                    # fits now, outgrows the pool while decoding
    s.add(grows)
    run(s)
    assert grows.done and isinstance(grows.error, RequestDoesNotFit) and grows.num_generated == 2
    assert cache.num_free_pages() == 2 and cache.num_free_slots == 4


def test_waiting_head_blocks_until_pages_free_up():
    s, cache = make(pages=4, page=4, budget=64)
    a, b = req(0, 12, max_tokens=2), req(1, 8, max_tokens=2)
    s.add(a); s.add(b)
    plan = s.schedule()
    assert shape(plan) == [(0, 12)] and list(s.waiting) == [b]
    assert not cache.holds(1)                                          # it holds nothing while it waits
    run(s)
    assert a.done and b.done and b.error is None


def test_shared_prefix_counts_cached_tokens_once():
    s, cache = make(pages=16, page=4, budget=64, sharing=True)
    a = req(0, 10, max_tokens=1)
    s.add(a)
    run(s)
    b = req(1, 10, max_tokens=1)
    b.tokens = list(a.tokens[:10])
    s.add(b)
    plan = s.schedule()
    assert shape(plan) == [(1, 2)] and b.stats.cached_tokens == 8
    assert s.prefix_hit_tokens == 8 and s.prompt_tokens_total == 20


def test_abort_and_fail_all_release_everything():
    s, cache = make()
    a, b, c = req(0, 5), req(1, 5), req(2, 5)
    for r in (a, b, c):
        s.add(r)
    s.computed(s.schedule())
    s.abort(a)
    assert a.stats.finish_reason == "abort" and not cache.holds(0)
    failed = s.fail_all(RuntimeError("boom"))
    assert {r.rid for r in failed} == {1, 2} and all(isinstance(r.error, RuntimeError) for r in failed)
    assert cache.num_free_pages() == cache.num_pages and cache.num_free_slots == 4
    cache.check()


def test_plan_is_typed_and_names_what_happened():
    s, cache = make(pages=4, page=4, budget=64)
    a, b = req(0, 6, max_tokens=8), req(1, 6, max_tokens=8, first=50)
    s.add(a); s.add(b)
    plan = s.schedule()
    assert isinstance(plan, Plan) and plan.admitted == [a, b] and plan.num_tokens == 12
    assert [(sl.start, sl.count, sl.wants_logits) for sl in plan] == [(0, 6, True), (0, 6, True)]
    assert plan.kinds() == (0, 12)
    s.computed(plan)
    s.accept(a, 7); s.accept(b, 7)
    plan = s.schedule()
    assert plan.kinds() == (2, 0) and not plan.preempted
    s.computed(plan)
    s.accept(a, 7); s.accept(b, 7)
    plan = s.schedule()                                  # position 7 of both: the last place in their pages
    s.computed(plan)
    s.accept(a, 7); s.accept(b, 7)
    plan = s.schedule()                                  # a needs a third page: b, the newest, gives way
    assert plan.preempted == [b] and shape(plan) == [(0, 1)] and list(s.waiting) == [b] and b.num_computed == 0


def test_preemption_policy_is_a_parameter():
    """With "least_computed" the request that is cheapest to recompute gives way, not the newest."""
    for policy, victim in (("newest", 1), ("least_computed", 0), (lambda running: running[0], 0)):
        s, cache = make(pages=6, page=4, budget=64, preemption=policy)
        a, b = req(0, 3, max_tokens=20), req(1, 13, max_tokens=20, first=50)
        s.add(a); s.add(b)
        gone = []
        for _ in range(12):
            plan = s.schedule()
            gone += [r.rid for r in plan.preempted]
            if gone:
                break
            s.computed(plan)
            for sl in plan:
                if sl.wants_logits:
                    s.accept(sl.request, 9)
        assert gone == [victim], policy
        cache.check()


def test_window_prompt_is_cut_to_the_room_there_is():
    """Window 24, pages of 8, a pool of 6 pages, a prompt of 200 tokens under a budget of 128: a portion of
    128 would need pages for window + 128 tokens; the request is alone, so its portions are cut to the
    room the pool has (48 tokens first, then what the passed pages give back) instead of failing."""
    s, cache = make(pages=6, page=8, budget=128, max_len=512, window=24)
    r = req(0, 200, max_tokens=3)
    s.add(r)
    plans = run(s)
    assert r.error is None and r.done and r.num_generated == 3
    sizes = [n for p in plans for rid, n in p]
    assert sizes[0] == 48 and sum(sizes[:-2]) == 200 and max(sizes) <= 48 and s.preemptions == 0
    assert cache.num_free_pages() == 6
    # two such requests: the older one is served, the newer one waits or gives way, both finish
    s, cache = make(pages=6, page=8, budget=128, max_len=512, window=24)
    a, b = req(0, 150, max_tokens=2), req(1, 90, max_tokens=2, first=500)
    s.add(a); s.add(b)
    run(s)
    assert a.error is None and b.error is None and a.num_generated == 2 and b.num_generated == 2
    assert cache.num_free_pages() == 6
