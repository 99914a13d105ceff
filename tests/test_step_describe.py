"""The step function's description of a batch (no GPU): sections, planners, and what is kept between steps."""
from types import SimpleNamespace

import numpy as np
import torch

from qwen_inference_lab_b200.cache import CacheManager
from qwen_inference_lab_b200.engine import StepEntry, StepRunner
from qwen_inference_lab_b200.parts import KVCacheSpec, LayerCall, StepPlanner
from qwen_inference_lab_b200.parts.attention import PagedAttentionPlanner


class FakeModel:
    """Just what ``StepRunner`` asks of a model before anything runs."""
    device, dtype = torch.device("cpu"), torch.float32
    vocab_size, max_positions = 1000, 4096
    order = [LayerCall(0)]

    def __init__(self, planners):
        self._planners = planners

    def cache_specs(self):
        return [KVCacheSpec(1, 8)]

    def is_graph_safe(self):
        return False

    def step_planners(self):
        return {p.key: p for p in self._planners}


def make(planners=None, pages=64, page_size=4, rows=4):
    model = FakeModel(planners if planners is not None else [PagedAttentionPlanner()])
    cache = CacheManager(model.cache_specs(), num_pages=pages, page_size=page_size, max_requests=rows,
                         max_context=model.max_positions, dtype=torch.float32, device="cpu")
    return cache, StepRunner(model, cache, use_graphs=False)


def section(description, name):
    begin, count = description.offsets[name]
    return description.packed[begin:begin + count].tolist()


def advance(cache, entries):
    for e in entries:
        end = cache.written(e.request_id) + len(e.tokens)
        cache.ensure(e.request_id, end)
        cache.advance(e.request_id, end)


def test_sections_of_a_mixed_batch():
    cache, runner = make()
    cache.admit("a"); cache.admit("b"); cache.admit("c")
    advance(cache, [StepEntry("b", list(range(10)))])
    entries = [StepEntry("a", list(range(1, 151)), [149]), StepEntry("b", [7], [0]), StepEntry("c", [1, 2, 3], [0, 2])]
    d = runner._describe(entries)
    assert d.segments.n_tokens == 154 and d.max_context == 150
    assert section(d, "seg_row") == [0, 1, 2] and section(d, "seg_start") == [0, 150, 151]
    assert section(d, "seg_len") == [150, 1, 3] and section(d, "seg_pos0") == [0, 10, 0]
    assert section(d, "positions")[148:154] == [148, 149, 10, 0, 1, 2]
    assert section(d, "token_row")[148:154] == [0, 0, 1, 2, 2, 2]
    assert section(d, "logit_rows") == [149, 150, 151, 153]
    tiles = np.array(section(d, "paged_attention.tile_info")).reshape(-1, 4).tolist()
    assert tiles == [[128, 128, 22, 0], [64, 64, 64, 0], [0, 0, 64, 0], [151, 0, 3, 2]]     # longest contexts first
    assert np.array(section(d, "paged_attention.big_tile_info")).reshape(-1, 4).tolist() == [[0, 0, 128, 0]]
    assert np.array(section(d, "paged_attention.rest_tile_info")).reshape(-1, 4).tolist() == [[128, 128, 22, 0], [151, 0, 3, 2]]
    assert section(d, "paged_attention.decode_info") == [150, 10, 1, 11]
    assert d.offsets["feed"][1] == 0 and all(begin % 4 == 0 for begin, _ in d.offsets.values())


def test_a_readmitted_id_is_described_with_its_new_row():
    """What is kept from one all-single-token step to the next holds block-table rows: an id that was
    released and admitted again (trace replay does that) sits in another row and must not run with the old one."""
    cache, runner = make()
    cache.admit("a")
    advance(cache, [StepEntry("a", [1, 2, 3])])
    first = runner._describe([StepEntry("a", [5], [0])])
    assert section(first, "token_row") == [0] and section(first, "paged_attention.decode_info") == [0, 3, 0, 4]
    advance(cache, [StepEntry("a", [5])])
    cache.release("a")
    cache.admit("b")                      # takes the next free row: 1
    cache.admit("a")                      # and "a" comes back in row 2
    assert cache.rows == {"b": 1, "a": 2}
    advance(cache, [StepEntry("a", [1, 2, 3])])       # a portion first (the general description), then single tokens
    runner._describe([StepEntry("a", [9, 9], [])])
    again = runner._describe([StepEntry("a", [5], [0])])
    assert section(again, "token_row") == [2] and section(again, "seg_row") == [2]
    assert section(again, "paged_attention.decode_info") == [0, 3, 2, 4]
    # the same id in the same row: the kept description is refreshed in place, positions move on
    advance(cache, [StepEntry("a", [5])])
    third = runner._describe([StepEntry("a", [6], [0])])
    assert third.packed is again.packed and section(third, "token_ids") == [6]
    assert section(third, "positions") == [4] and section(third, "paged_attention.decode_info") == [0, 4, 2, 5]
    assert third.max_context == 5 and third.segments.starts.tolist() == [4]


def test_single_token_sections_depend_on_the_number_of_requests_only():
    """Recorded graphs hold the offsets of a step's sections: for steps of single tokens they may not move
    with positions or rows."""
    cache, runner = make(rows=4, pages=256)
    for rid, length in (("a", 3), ("b", 90), ("c", 17)):
        cache.admit(rid)
        advance(cache, [StepEntry(rid, list(range(length)))])
    one = runner._describe([StepEntry(r, [1], [0]) for r in "abc"])
    offsets_one = dict(one.offsets)
    advance(cache, [StepEntry(r, [1]) for r in "abc"])
    cache.release("b"); cache.admit("d"); advance(cache, [StepEntry("d", list(range(300)))])
    two = runner._describe([StepEntry(r, [1], [0]) for r in "adc"])
    assert two.offsets == offsets_one and two.packed is not one.packed


def test_a_planner_of_the_tests_own_gets_its_sections_and_a_refresh_refusal_plans_again():
    class Chunks(StepPlanner):
        key = "chunks_of_5"
        calls = 0

        def plan(self, segments):
            Chunks.calls += 1
            cuts = [(int(f) + off, min(5, int(n) - off)) for f, n in zip(segments.first, segments.lens)
                    for off in range(0, int(n), 5)]
            return dict(cuts=np.array(cuts).reshape(-1), count=np.array([len(cuts)]))

    cache, runner = make([PagedAttentionPlanner(), Chunks()])
    cache.admit("a"); cache.admit("b")
    d = runner._describe([StepEntry("a", list(range(12))), StepEntry("b", [4])])
    assert section(d, "chunks_of_5.cuts") == [0, 5, 5, 5, 10, 2, 12, 1] and section(d, "chunks_of_5.count") == [4]
    runner._meta_dev[:len(d.packed)] = torch.from_numpy(d.packed)
    ctx = runner._context(d)
    assert ctx.plans["chunks_of_5"].count == dict(cuts=8, count=1)
    assert ctx.plans["chunks_of_5"].array["cuts"].tolist() == [0, 5, 5, 5, 10, 2, 12, 1]
    assert ctx.plans["paged_attention"].count["decode_info"] == 4
    advance(cache, [StepEntry("a", list(range(12))), StepEntry("b", [4])])
    before = Chunks.calls
    runner._describe([StepEntry("a", [1], [0]), StepEntry("b", [1], [0])])
    advance(cache, [StepEntry("a", [1]), StepEntry("b", [1])])
    runner._describe([StepEntry("a", [1], [0]), StepEntry("b", [1], [0])])      # Chunks cannot refresh: planned again
    assert Chunks.calls == before + 2
