"""The scheduler's decisions (no GPU): admission, portions under a budget, fairness, finishing."""
import pytest
import torch

from qwen_inference_lab_b200.cache import CacheManager
from qwen_inference_lab_b200.engine.scheduler import Scheduler, Sequence
from qwen_inference_lab_b200.parts import KVCacheSpec


def make(pages=16, page_size=4, max_active=4, budget=8, chunk=4):
    cache = CacheManager([KVCacheSpec(1, 4)], num_pages=pages, page_size=page_size, max_requests=max_active,
                         max_context=256, dtype=torch.float32, device="cpu", max_step_tokens=budget)
    return cache, Scheduler(cache, token_budget=budget, prefill_chunk=chunk, max_active=max_active)


def request(rid, prompt_len, new=4):
    return Sequence(rid, list(range(1, prompt_len + 1)), new, set(), 0.0)


def shape(plan):
    return [(turn.sequence.id, turn.start, turn.count) for turn in plan]


def run(cache, scheduler, plan):
    """What the engine does with a plan: the step takes pages and moves the cache's progress, the scheduler
    is told that the turns are queued, and the tokens the step chose are read at once (no running ahead)."""
    for turn in plan:
        end = turn.start + turn.count
        cache.ensure(turn.sequence.id, end)
        cache.advance(turn.sequence.id, end)
    scheduler.queued(plan)
    for turn in plan:
        if turn.samples:
            scheduler.read(turn.sequence, 100 + len(turn.sequence.output), 0.0)


def test_prompts_are_cut_into_portions_under_the_budget_then_decoded():
    cache, scheduler = make(budget=8, chunk=4)
    scheduler.add(request(0, 10)); scheduler.add(request(1, 3))
    plan = scheduler.plan()
    assert shape(plan) == [(0, 0, 4), (1, 0, 3)]
    run(cache, scheduler, plan)
    plan = scheduler.plan()         # request 1 now decodes one token; request 0 continues its prompt
    assert shape(plan) == [(0, 4, 4), (1, 3, 1)]
    assert plan[1].entry.tokens == [100] and plan[1].samples and not plan[0].samples
    run(cache, scheduler, plan)
    plan = scheduler.plan()
    assert shape(plan) == [(0, 8, 2), (1, 4, 1)]


def test_budget_smaller_than_a_portion_and_round_robin_fairness():
    cache, scheduler = make(budget=5, chunk=4, max_active=3)
    for rid in range(3):
        scheduler.add(request(rid, 9, new=2))
    served = []
    for _ in range(6):
        plan = scheduler.plan()
        assert sum(turn.count for turn in plan) <= 5
        served.append([(turn.sequence.id, turn.count) for turn in plan])
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
    assert [turn.sequence.id for turn in plan] == [0, 2]
    assert scheduler.table[1].state == "waiting" and [s.id for s in scheduler.queue] == [1]
    assert cache.unreserved == 0
    run(cache, scheduler, plan)
    for _ in range(3):                        # request 2 finishes after 4 tokens and frees its credit
        run(cache, scheduler, scheduler.plan())
    assert scheduler.table[2].state == "completed"
    plan = scheduler.plan()                   # still no room: 6 + 3 > 8
    assert [turn.sequence.id for turn in plan] == [0]
    run(cache, scheduler, plan)
    assert scheduler.table[0].state == "completed"
    plan = scheduler.plan()
    assert [turn.sequence.id for turn in plan] == [1]
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
        assert len(scheduler.ring) <= 4
        steps += 1
        assert steps < 500
    assert all(r.state == "completed" for r in scheduler.table.values())
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
    """A token that a queued step has chosen and the host has not read counts as input: the next plan feeds
    its place (marked -1) from the row it has in the device buffer, and a request whose unread token is its
    last gets no further work."""
    cache, scheduler = make(budget=8, chunk=4)
    scheduler.add(request(0, 3, new=2)); scheduler.add(request(1, 6, new=3))
    tokens = lambda plan: [(t.sequence.id, t.start, t.entry.tokens, t.entry.want, t.entry.feed) for t in plan]
    plan = scheduler.plan()
    assert tokens(plan) == [(0, 0, [1, 2, 3], [2], None), (1, 0, [1, 2, 3, 4], [], None)]
    scheduler.queued(plan)                      # request 0's first token is now on the device, in row 0
    r0, r1 = scheduler.table[0], scheduler.table[1]
    assert (r0.fed, r0.unread, r0.feed_row, r1.fed, r1.unread) == (3, 1, 0, 4, 0)
    assert r0.input_length == 4 and r0.tokens_from(2, 2) == [3, -1] and r0.tokens_from(3, 1) == [-1]
    plan = scheduler.plan()                     # request 0 decodes the unread token, request 1 ends its prompt
    assert tokens(plan) == [(0, 3, [-1], [0], 0), (1, 4, [5, 6], [1], None)]
    scheduler.queued(plan)                      # both leave a token on the device: rows 0 and 1
    assert (r0.unread, r1.unread, r1.feed_row) == (2, 1, 1)
    assert scheduler.read(r0, 55, 1.0) == dict(request_id=0, token_id=55, timestamp_s=1.0, finished=False)
    assert r0.unread == 1 and r0.awaits_last_token and not r1.awaits_last_token
    plan = scheduler.plan()                     # request 0 waits for its last token, request 1 goes on
    assert tokens(plan) == [(1, 6, [-1], [0], 1)]
    scheduler.queued(plan)
    assert scheduler.read(r0, 56, 2.0)["finished"] and r0.state == "completed" and r0.finish_reason == "length"
    assert [s.id for s in scheduler.ring] == [1]
    assert scheduler.read(r0, 57, 3.0) is None  # a token for a request that has ended is dropped
    # nothing to plan while the only active request waits for its last token, and no complaint about it
    scheduler.read(r1, 7, 3.0)
    plan = scheduler.plan()
    assert tokens(plan) == [(1, 7, [-1], [0], 0)]
    scheduler.queued(plan)
    scheduler.read(r1, 8, 4.0)
    assert r1.output == [7, 8] and r1.unread == 1
    scheduler.add(request(2, 40, new=20))       # fits the cache, but not beside request 1: waits
    assert r1.awaits_last_token and scheduler.plan() == [] and [s.id for s in scheduler.queue] == [2]
    assert scheduler.read(r1, 9, 5.0)["finished"]
    assert shape(scheduler.plan()) == [(2, 0, 4)]


def test_an_end_token_stops_a_request_and_counts_before_length():
    cache, scheduler = make()
    sequence = Sequence(0, [1, 2, 3], 2, {9}, 10.0)
    scheduler.add(sequence)
    run_plan = scheduler.plan()
    scheduler.queued(run_plan)
    assert not scheduler.read(sequence, 4, 10.5)["finished"]
    scheduler.queued(scheduler.plan())
    event = scheduler.read(sequence, 9, 11.5)       # the end token arrives as the last allowed token: "eos" wins
    assert event["finished"] and sequence.finish_reason == "eos" and sequence.output == [4, 9]
    report = sequence.report()
    assert report["ttft_s"] == 0.5 and report["e2e_s"] == 1.5 and report["tpot_s"] == 1.0
    assert report["token_times_s"] == [0.5, 1.5] and report["state"] == "completed"
    assert scheduler.idle and cache.free_pages() == 16
