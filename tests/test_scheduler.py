"""The scheduler's decisions (no GPU): admission, portions under a budget, fairness, finishing."""
import pytest
import torch

from qwen_inference_lab_b200.cache import CacheManager
from qwen_inference_lab_b200.engine.scheduler import Request, Scheduler
from qwen_inference_lab_b200.parts import KVCacheSpec


def make(pages=16, page_size=4, max_active=4, budget=8, chunk=4):
    cache = CacheManager([KVCacheSpec(1, 4)], num_pages=pages, page_size=page_size, max_requests=max_active,
                         max_context=256, dtype=torch.float32, device="cpu", max_step_tokens=budget)
    return cache, Scheduler(cache, token_budget=budget, prefill_chunk=chunk, max_active=max_active)


def request(rid, prompt_len, new=4):
    return Request(rid, list(range(1, prompt_len + 1)), new, set(), 0.0)


def run(cache, scheduler, work):
    """What the engine does after a step: pages, progress, one generated token when the input is consumed."""
    for item in work:
        r = scheduler.requests[item.request_id]
        cache.ensure(r.id, item.start + len(item.tokens))
        cache.advance(r.id, item.start + len(item.tokens))
        r.computed = item.start + len(item.tokens)
        if r.computed == len(r.input_tokens):
            r.output.append(100 + len(r.output))
            if len(r.output) == r.max_new_tokens:
                scheduler.retire(r.id, "completed", "length")


def test_prompts_are_cut_into_portions_under_the_budget_then_decoded():
    cache, scheduler = make(budget=8, chunk=4)
    scheduler.add(request(0, 10)); scheduler.add(request(1, 3))
    plan = scheduler.plan()
    assert [(w.request_id, w.start, len(w.tokens)) for w in plan] == [(0, 0, 4), (1, 0, 3)]
    run(cache, scheduler, plan)
    plan = scheduler.plan()         # request 1 now decodes one token; request 0 continues its prompt
    assert [(w.request_id, w.start, len(w.tokens)) for w in plan] == [(0, 4, 4), (1, 3, 1)]
    assert plan[1].tokens == [100]
    run(cache, scheduler, plan)
    plan = scheduler.plan()
    assert [(w.request_id, w.start, len(w.tokens)) for w in plan] == [(0, 8, 2), (1, 4, 1)]


def test_budget_smaller_than_a_portion_and_round_robin_fairness():
    cache, scheduler = make(budget=5, chunk=4, max_active=3)
    for rid in range(3):
        scheduler.add(request(rid, 9, new=2))
    served = []
    for _ in range(6):
        plan = scheduler.plan()
        assert sum(len(w.tokens) for w in plan) <= 5
        served.append([(w.request_id, len(w.tokens)) for w in plan])
        run(cache, scheduler, plan)
    # whoever was cut short or not reached comes first next time: nobody starves
    assert served[0] == [(0, 4), (1, 1)]
    assert served[1] == [(2, 4), (0, 1)]
    assert served[2] == [(1, 4), (2, 1)]
    ids = [rid for plan in served for rid, _ in plan]
    assert all(ids.count(r) >= 3 for r in range(3))


def test_max_active_and_admission_by_reservation():
    cache, scheduler = make(pages=8, page_size=4, max_active=2, budget=64, chunk=64)
    scheduler.add(request(0, 20, new=5))      # 24 cached tokens: 6 pages
    scheduler.add(request(1, 12, new=1))      # 12 tokens: 3 pages, does not fit beside request 0
    scheduler.add(request(2, 5, new=4))       # 8 tokens: 2 pages, overtakes request 1
    plan = scheduler.plan()
    assert [w.request_id for w in plan] == [0, 2]
    assert scheduler.requests[1].state == "waiting" and list(scheduler.waiting) == [1]
    assert cache.unreserved == 0
    run(cache, scheduler, plan)
    for _ in range(3):                        # request 2 finishes after 4 tokens and frees its credit
        run(cache, scheduler, scheduler.plan())
    assert scheduler.requests[2].state == "completed"
    plan = scheduler.plan()                   # still no room: 6 + 3 > 8
    assert [w.request_id for w in plan] == [0]
    run(cache, scheduler, plan)
    assert scheduler.requests[0].state == "completed"
    plan = scheduler.plan()
    assert [w.request_id for w in plan] == [1]
    cache.check_invariants()


def test_a_request_that_can_never_fit_is_refused_at_once():
    cache, scheduler = make(pages=4, page_size=4)
    with pytest.raises(ValueError, match="capacity"):
        scheduler.add(request(0, 14, new=4))            # 17 cached tokens > 16
    scheduler.add(request(1, 13, new=4))                # 16 cached tokens: exactly fits
    assert not scheduler.idle
    with pytest.raises(ValueError, match="duplicate"):
        scheduler.add(request(1, 2))


def test_pages_never_run_out_in_mid_flight():
    """Every admitted request can always take its next portion: the pool is only ever promised once."""
    cache, scheduler = make(pages=12, page_size=2, max_active=4, budget=7, chunk=3)
    for rid in range(9):
        scheduler.add(request(rid, 3 + rid, new=3))
    steps = 0
    while not scheduler.idle:
        plan = scheduler.plan()
        assert plan, "a non-idle scheduler always has work"
        run(cache, scheduler, plan)          # ensure() inside would raise if pages ran out
        cache.check_invariants()
        assert len(scheduler.active) <= 4
        steps += 1
        assert steps < 500
    assert all(r.state == "completed" for r in scheduler.requests.values())
    assert cache.free_pages() == 12 and not cache.owners()


def test_retire_is_idempotent_and_frees_only_active_requests():
    cache, scheduler = make(max_active=1)
    scheduler.add(request(0, 4)); scheduler.add(request(1, 4))
    run(cache, scheduler, scheduler.plan())
    assert scheduler.retire(1, "cancelled", "cancelled")        # waiting: nothing to free
    assert scheduler.retire(0, "cancelled", "cancelled") and not scheduler.retire(0, "cancelled", "cancelled")
    assert scheduler.idle and cache.free_pages() == 16 and scheduler.plan() == []


def test_budgets_must_be_positive_integers():
    cache, _ = make()
    for bad in (dict(token_budget=0), dict(prefill_chunk=-1), dict(max_active=1.5)):
        with pytest.raises(ValueError):
            Scheduler(cache, **bad)


def test_planning_a_step_ahead_of_the_tokens():
    """A token that a queued step has sampled and the host has not read counts as input: the next plan feeds
    its place (marked -1) back, and a request whose pending token is its last gets no further work."""
    cache, scheduler = make(budget=8, chunk=4)
    scheduler.add(request(0, 3, new=2)); scheduler.add(request(1, 6, new=3))
    plan = scheduler.plan()
    assert [(w.request_id, w.start, w.tokens) for w in plan] == [(0, 0, [1, 2, 3]), (1, 0, [1, 2, 3, 4])]
    r0, r1 = scheduler.requests[0], scheduler.requests[1]
    r0.computed, r1.computed = 3, 4
    r0.pending = 1                              # request 0's first token is on the device
    assert r0.input_length == 4 and r0.input_slice(2, 2) == [3, -1] and r0.input_slice(3, 1) == [-1]
    plan = scheduler.plan()                     # request 0 decodes the unread token, request 1 ends its prompt
    assert [(w.request_id, w.start, w.tokens) for w in plan] == [(0, 3, [-1]), (1, 4, [5, 6])]
    r0.output.append(55)                        # read now; the step just planned has sampled the second
    r0.computed, r1.computed, r1.pending = 4, 6, 1
    assert r0.pending == 1 and r0.ends_with_pending and not r1.ends_with_pending
    plan = scheduler.plan()                     # request 0 waits for its last token, request 1 goes on
    assert [(w.request_id, w.start, w.tokens) for w in plan] == [(1, 6, [-1])]
    r0.output.append(56); r0.pending = 0
    scheduler.retire(0, "completed", "length")
    assert list(scheduler.active) == [1]
    # nothing to plan while the only active request waits for its last token, and no complaint about it
    r1.output += [7, 8]; r1.computed = 8; r1.pending = 1
    scheduler.add(request(2, 40, new=20))       # fits the cache, but not beside request 1: waits
    assert r1.ends_with_pending and scheduler.plan() == [] and list(scheduler.waiting) == [2]
