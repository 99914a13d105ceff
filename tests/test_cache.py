"""The cache manager's bookkeeping (no GPU): pages, block tables, windows, state slots."""
import random

import pytest
import torch

from qwen_inference_lab_b200.cache import CacheError, CacheManager, OutOfPages
from qwen_inference_lab_b200.parts import KVCacheSpec, StateSpec

FULL = KVCacheSpec(kv_heads=2, head_dim=4)
WINDOWED = KVCacheSpec(kv_heads=1, head_dim=4, window=10)
STATE = StateSpec(shape=(3, 2), dtype=torch.float32)


def manager(specs=(FULL, FULL), pages=8, page_size=4, max_requests=4, max_context=64, **kw):
    return CacheManager(list(specs), num_pages=pages, page_size=page_size, max_requests=max_requests,
                        max_context=max_context, dtype=torch.float32, device="cpu", **kw)


def test_reservations_take_credit_not_pages():
    cache = manager()
    assert cache.admit("a", 14)                 # 4 pages of credit
    assert cache.free_pages() == 8 and cache.unreserved == 4
    assert cache.admit("b", 16) and cache.unreserved == 0
    assert not cache.admit("c", 1)              # no credit left: waits, nothing changed
    assert "c" not in cache.rows and len(cache.free_rows) == 2
    cache.ensure("a", 5)
    assert cache.free_pages() == 6 and cache.written("a") == 0
    cache.advance("a", 5)
    cache.release("b")
    assert cache.admit("c", 16)
    cache.check_invariants()


def test_tables_need_not_be_contiguous_and_mirror_the_device():
    cache = manager(pages=6)
    cache.admit("a", 8); cache.admit("b", 8)
    cache.ensure("a", 4); cache.ensure("b", 4); cache.ensure("a", 8)
    group = cache.kv_groups[0]
    assert group.tables["a"] == [0, 2] and group.tables["b"] == [1]
    cache.flush_tables()
    row = cache.row("a")
    assert group.dev_table[row, :2].tolist() == [0, 2] and group.dev_table[row, 2:].eq(-1).all()
    views = cache.views()
    assert views[0].pages.shape == (6, 2, 2, 4, 4) and views[0].block_table is views[1].block_table
    assert views[0].pages.data_ptr() != views[1].pages.data_ptr()      # one plane per layer, shared page ids


def test_rules_are_enforced():
    cache = manager()
    with pytest.raises(CacheError):
        cache.ensure("nobody", 1)
    with pytest.raises(CacheError):
        cache.release("nobody")
    cache.admit("a", 6)
    with pytest.raises(CacheError):
        cache.admit("a", 6)                     # duplicate owner
    with pytest.raises(CacheError):
        cache.admit("z", 0)
    with pytest.raises(CacheError):
        cache.ensure("a", 7)                    # beyond the reservation
    with pytest.raises(CacheError):
        cache.ensure("a", 0)
    cache.ensure("a", 6); cache.advance("a", 6)
    with pytest.raises(CacheError):
        cache.advance("a", 3)                   # progress cannot go back
    cache.release("a")
    with pytest.raises(CacheError):
        cache.release("a")                      # freed twice
    assert cache.free_pages() == 8
    assert not cache.fits(8 * 4 + 1) and cache.fits(8 * 4)
    with pytest.raises(CacheError):
        manager(pages=0)


def test_unreserved_requests_grow_until_the_pool_is_empty():
    cache = manager(pages=3)
    assert cache.admit("a") and cache.admit("b")
    cache.ensure("a", 8); cache.advance("a", 8)
    cache.ensure("b", 4)
    with pytest.raises(OutOfPages):
        cache.ensure("a", 9)
    cache.check_invariants()
    cache.release("b")
    cache.ensure("a", 12)                       # the freed page is used again
    assert cache.kv_groups[0].tables["a"][-1] == 2
    cache.check_invariants()


def test_rows_run_out_before_pages():
    cache = manager(max_requests=2, pages=64)
    assert cache.admit(1, 4) and cache.admit(2, 4) and not cache.admit(3, 4)
    cache.release(1)
    assert cache.admit(3, 4) and cache.row(3) == 0


def test_window_groups_give_pages_back_as_the_window_passes():
    cache = manager(specs=(FULL, WINDOWED, WINDOWED), pages=16, max_context=64, max_step_tokens=8)
    assert len(cache.kv_groups) == 2 and cache.kv_groups[1].members == [1, 2]
    assert cache.admit("a", 40)
    full, windowed = cache.kv_groups
    assert full.reserved["a"] == 10 and windowed.reserved["a"] == 6     # ceil((10 + 8) / 4) + 1
    position = 0
    while position < 40:
        step = min(8, 40 - position)
        cache.ensure("a", position + step)
        position += step
        cache.advance("a", position)
        cache.check_invariants()
        live = [p for p in windowed.tables["a"] if p >= 0]
        assert len(live) <= 6
        first_needed = max(0, position - 10 + 1) // 4
        assert all(p == -1 for p in windowed.tables["a"][:first_needed])
        assert all(p >= 0 for p in windowed.tables["a"][first_needed:])
        assert all(p >= 0 for p in full.tables["a"])
    assert len(full.free) == 6 and len(windowed.free) == 16 - 3
    cache.release("a")
    assert len(full.free) == 16 and len(windowed.free) == 16
    cache.check_invariants()


def test_state_slots_are_zeroed_at_admission_and_follow_the_row():
    cache = manager(specs=(STATE, FULL, STATE), max_requests=2)
    assert len(cache.state_groups) == 1 and len(cache.kv_groups) == 1
    views = cache.views()
    assert views[0].slots.shape == (2, 3, 2) and views[2].slots.shape == (2, 3, 2)
    cache.admit("a", 4)
    views[0].slots[cache.row("a")] = 7.0
    views[2].slots[cache.row("a")] = 9.0
    cache.release("a")
    cache.admit("b", 4)
    assert cache.row("b") == 1
    cache.admit("c", 4)
    assert cache.row("c") == 0 and views[0].slots[0].eq(0).all() and views[2].slots[0].eq(0).all()


def test_state_that_belongs_to_requests_not_layers():
    cache = CacheManager([KVCacheSpec(1, 4)], num_pages=8, page_size=4, max_requests=3, max_context=64,
                         dtype=torch.float32, device="cpu", request_state={"sampler": StateSpec((4,), torch.int64)})
    slots = cache.request_state("sampler")
    assert slots.shape == (3, 4) and slots.dtype == torch.int64
    cache.admit("a"); cache.admit("b")
    slots[cache.row("b")] = torch.tensor([1, 2, 3, 4])
    cache.release("b")
    cache.admit("c"); cache.admit("d")            # "d" gets the row "b" had: zeroed again
    assert cache.row("d") == 1 and slots[1].tolist() == [0, 0, 0, 0]
    with pytest.raises(KeyError):
        cache.request_state("nothing")


def test_views_follow_the_order_of_a_model_that_shares_caches():
    from qwen_inference_lab_b200.parts import LayerCall
    cache = manager(specs=(FULL, None, FULL))
    order = [LayerCall(0), LayerCall(1, reads_cache_of=0), LayerCall(0)]
    views = cache.views(order)
    assert views[1].pages.data_ptr() == views[0].pages.data_ptr()
    assert views[2].pages.data_ptr() != views[0].pages.data_ptr()
    assert cache.views()[1] is None


@pytest.mark.parametrize("seed", range(6))
def test_no_page_is_lost_held_twice_or_freed_twice_under_random_traffic(seed):
    rng = random.Random(seed)
    cache = manager(specs=(FULL, WINDOWED), pages=24, page_size=rng.choice([1, 3, 4]), max_requests=5,
                    max_context=200, max_step_tokens=16)
    live, next_id = {}, 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            limit = rng.choice([None, rng.randint(1, 60)])
            if cache.admit(next_id, limit):
                live[next_id] = dict(limit=limit, done=0)
            next_id += 1
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            state = live[rid]
            room = (state["limit"] or 80) - state["done"]
            if room <= 0:
                continue
            count = rng.randint(1, min(16, room))
            try:
                cache.ensure(rid, state["done"] + count)
            except OutOfPages:
                assert state["limit"] is None      # reserved requests never run dry
                continue
            state["done"] += count
            cache.advance(rid, state["done"])
        elif live:
            rid = rng.choice(list(live))
            cache.release(rid)
            del live[rid]
        cache.check_invariants()
    for rid in list(live):
        cache.release(rid)
    cache.check_invariants()
    assert all(len(g.free) == g.capacity for g in cache.kv_groups) and len(cache.free_rows) == 5
