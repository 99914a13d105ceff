"""Replay of the same requests under four ways of cutting the work, against the plain implementation."""
import pytest
import torch

from tests import harness
from tests.tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D

pytestmark = pytest.mark.gpu

CASES = {
    "A": dict(cfg=TINY_A, seed=0, page_size=4, lengths=(5, 17, 33, 90, 41, 12)),
    "B": dict(cfg=TINY_B, seed=1, page_size=8, lengths=(1, 9, 31, 64, 100, 150)),
    "C": dict(cfg=TINY_C, seed=2, page_size=16, lengths=(40, 3, 130, 70, 25, 90)),
    "D": dict(cfg=TINY_D, seed=3, page_size=16, lengths=(700, 300, 1100, 130, 520)),
}
SCHEDULES = {
    "whole": harness.whole_schedule,
    "tail_decode": harness.tail_decode_schedule,
    "chunks": harness.chunk_schedule,
    "mixed": harness.mixed_schedule,
}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    result = {}
    for name, case in CASES.items():
        folder = tmp_path_factory.mktemp(f"tiny{name}")
        weights = harness.write_folder(case["cfg"], case["seed"], folder)
        requests = {f"r{i}": harness.random_tokens(case["cfg"], n, 50 + i) for i, n in enumerate(case["lengths"])}
        result[name] = (folder, weights, requests)
    return result


def pool_for(schedule_name, requests, page_size):
    """Pages of the pool: what the schedule holds at its peak and one page more, so that the free list
    (first in, first out) is walked through again and again and released pages come back to other requests."""
    schedule = SCHEDULES[schedule_name](requests)
    return schedule, harness.peak_pages(schedule, page_size) + 1


def replay(folders, case, schedule_name, dtype):
    folder, weights, requests = folders[case]
    page_size = CASES[case]["page_size"]
    schedule, num_pages = pool_for(schedule_name, requests, page_size)
    _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=num_pages, page_size=page_size)
    ledger = harness.PageLedger(cache)
    actual = harness.run_schedule(runner, cache, schedule, ledger)
    assert cache.free_pages() == num_pages and not cache.owners()
    assert ledger.peak_held == num_pages - 1
    # every schedule runs more requests than the pool holds at once: pages must have changed hands, and the
    # mixed one hands them over while other requests are in the middle of theirs
    assert ledger.handovers > 0, "no page was used again by another request: the pool is too large"
    return actual


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", list(SCHEDULES))
@pytest.mark.parametrize("case", list(CASES))
def test_replay_matches_plain(folders, case, schedule, dtype):
    folder, weights, requests = folders[case]
    cfg = CASES[case]["cfg"]
    actual = replay(folders, case, schedule, dtype)
    expected = harness.plain_rows(requests, weights, cfg, torch.float32)
    yardstick = harness.plain_rows(requests, weights, cfg, dtype) if dtype == torch.bfloat16 else None
    harness.assert_rows_close(actual, expected, dtype, f"tiny {case} {schedule} {dtype}", yardstick)


@pytest.mark.parametrize("case", list(CASES))
def test_float32_rows_are_the_same_bits_under_every_schedule(folders, case):
    """In float32 every sum is taken in an order that depends on the position alone: how the tokens were cut into
    steps, what else was in the batch and which pages held the cache must not change a single bit."""
    runs = {name: replay(folders, case, name, torch.float32) for name in SCHEDULES}
    reference = runs["whole"]
    for name, rows in runs.items():
        assert set(rows) == set(reference)
        different = [key for key in sorted(rows, key=lambda k: (k[0], k[1])) if not torch.equal(rows[key], reference[key])]
        assert not different, (f"tiny {case}: {len(different)} rows of schedule {name} differ from the whole run, first "
                               f"{different[0]}, by {(rows[different[0]] - reference[different[0]]).abs().max():.3e}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("case,length,tail", [("C", 540, 45), ("D", 1045, 50)])
def test_decoding_across_a_context_bucket_of_the_recorded_graphs(folders, case, length, tail, dtype):
    """Single-token steps are recorded per context bucket (512, 1024, ...): decoding from below a bucket's edge
    to above it switches to another recording with other span bounds in the attention."""
    folder, weights, _ = folders[case]
    cfg, page_size = CASES[case]["cfg"], CASES[case]["page_size"]
    requests = {"long": harness.random_tokens(cfg, length, 77), "short": harness.random_tokens(cfg, tail + 9, 78)}
    # both decode together, one token a step each: "long" crosses the edge, "short" stays far below it
    schedule = [([("long", requests["long"][:length - tail], []), ("short", requests["short"][:9], [])], [])]
    for i in range(tail):
        last = i == tail - 1
        schedule.append(([("long", [requests["long"][length - tail + i]], [0]), ("short", [requests["short"][9 + i]], [0])],
                         ["long", "short"] if last else []))
    num_pages = harness.peak_pages(schedule, page_size) + 1
    _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=num_pages, page_size=page_size)
    actual = harness.run_schedule(runner, cache, schedule)
    assert len({key[1] for key in runner._graphs}) == 2, "the run should have used two context buckets"
    expected_all = harness.plain_rows(requests, weights, cfg, torch.float32)
    expected = {k: expected_all[k] for k in actual}
    yardstick = None
    if dtype == torch.bfloat16:
        full = harness.plain_rows(requests, weights, cfg, dtype)
        yardstick = {k: full[k] for k in actual}
    harness.assert_rows_close(actual, expected, dtype, f"tiny {case} across a bucket {dtype}", yardstick)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B"])
def test_an_ended_id_admitted_again_runs_in_its_new_row(folders, case, dtype):
    """"a" ends and comes back while "b" is live, so it gets another block-table row; portions first, then single
    tokens (whose description the step function keeps from step to step)."""
    folder, weights, _ = folders[case]
    cfg, page_size = CASES[case]["cfg"], CASES[case]["page_size"]
    first, second, other = (harness.random_tokens(cfg, n, 90 + i) for i, n in enumerate((21, 30, 60)))
    schedule = [([("a", first[:16], list(range(16))), ("b", other[:7], list(range(7)))], [])]
    schedule += [([("a", [first[i]], [0]), ("b", [other[i - 9]], [0])], ["a"] if i == 20 else []) for i in range(16, 21)]
    schedule += [([("b", other[12:30], list(range(18))), ("a", second[:9], list(range(9)))], [])]      # "a" again
    schedule += [([("a", [second[i]], [0]), ("b", [other[i + 21]], [0])], []) for i in range(9, 30)]
    schedule += [([("b", other[51:], list(range(9)))], ["a", "b"])]
    _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=40, page_size=page_size)
    rows_seen = []
    original_admit = cache.admit
    cache.admit = lambda rid, limit=None: (original_admit(rid, limit), rows_seen.append((rid, cache.rows[rid])))[0]
    ledger = harness.PageLedger(cache)
    first_life = harness.run_schedule(runner, cache, schedule[:6], ledger)         # up to the end of "a"
    second_life = harness.run_schedule(runner, cache, schedule[6:], ledger)
    assert [r for rid, r in rows_seen if rid == "a"] == [0, 2]
    names = {"a1": first, "a2": second, "b": other}
    plain_all = harness.plain_rows(names, weights, cfg, torch.float32)
    plain_low = harness.plain_rows(names, weights, cfg, dtype) if dtype == torch.bfloat16 else None
    for actual, life in ((first_life, "a1"), (second_life, "a2")):
        rename = lambda key: (life, key[1]) if key[0] == "a" else key
        expected = {key: plain_all[rename(key)] for key in actual}
        yardstick = {key: plain_low[rename(key)] for key in actual} if plain_low else None
        harness.assert_rows_close(actual, expected, dtype, f"tiny {case} re-admitted id ({life}) {dtype}", yardstick)
    assert len(first_life) == 21 + 12 and len(second_life) == 30 + 48


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_a_neighbours_pages_do_not_reach_this_requests_logits(folders, dtype):
    """Two live requests share steps.  Whatever the neighbour's pages hold (its own keys and values, another
    sequence's, or NaN written over them), this request's logits keep every bit
    (tests/qil/test_batch_decode.py:76-90 of the reference)."""
    folder, weights, _ = folders["B"]
    cfg, page_size = CASES["B"]["cfg"], CASES["B"]["page_size"]
    mine = harness.random_tokens(cfg, 70, 5)
    neighbours = [harness.random_tokens(cfg, 70, 6), harness.random_tokens(cfg, 70, 7)]

    def run(neighbour, spoil):
        _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=24, page_size=page_size)
        from qwen_inference_lab_b200.engine import StepEntry
        cache.admit("me"); cache.admit("other")
        rows = []
        # portions side by side (pages of the two interleave), then single tokens side by side
        cuts = [(0, 13), (13, 40), (40, 41), (41, 42), (42, 43), (43, 60)] + [(i, i + 1) for i in range(60, 70)]
        for step, (lo, hi) in enumerate(cuts):
            if spoil and step >= 2:
                group = cache.kv_groups[0]
                pages = torch.tensor([p for p in group.tables["other"] if p >= 0], device="cuda")
                group.storage[:, pages] = float("nan")
                batch = [StepEntry("me", mine[lo:hi], list(range(hi - lo)))]       # the neighbour sits these steps out
            else:
                batch = [StepEntry("other", neighbour[lo:hi], []), StepEntry("me", mine[lo:hi], list(range(hi - lo)))]
            rows.append(runner.run(batch).float().cpu())
        held = cache.kv_groups[0].tables["me"]
        assert any(b - a != 1 for a, b in zip(held, held[1:])), "the two requests' pages should interleave"
        return torch.cat(rows)

    base = run(neighbours[0], spoil=False)
    assert torch.isfinite(base).all()
    assert torch.equal(base, run(neighbours[1], spoil=False)), "another neighbour changed this request's logits"
    spoiled = run(neighbours[0], spoil=True)
    assert torch.equal(base[:13 + 27], spoiled[:40])
    assert torch.isfinite(spoiled).all()
    # alone in its steps the request may take other kernels' paths in bfloat16 (rounding only); in float32: the same bits
    if dtype == torch.float32:
        assert torch.equal(base, spoiled)
    else:
        assert (base - spoiled).abs().max() < 0.05
    expected = harness.plain_rows({"me": mine}, weights, cfg, torch.float32)
    actual = {("me", p): base[p] for p in range(70)}
    yardstick = harness.plain_rows({"me": mine}, weights, cfg, dtype) if dtype == torch.bfloat16 else None
    harness.assert_rows_close(actual, expected, dtype, f"victim {dtype}", yardstick)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_recorded_steps_survive_a_step_that_outgrows_the_runner(folders, dtype):
    """Single-token steps are recorded as graphs; a later step with more tokens than the runner was
    made for replaces the buffers those graphs point into.  The recordings are then made anew, in a
    new memory pool, and the scratch that the parts keep between steps stays valid."""
    from qwen_inference_lab_b200.cache import CacheManager
    from qwen_inference_lab_b200.engine import StepRunner
    from qwen_inference_lab_b200.loading import load_model
    folder, weights, _ = folders["B"]
    cfg = CASES["B"]["cfg"]
    model = load_model(folder, device="cuda", dtype=dtype)
    cache = CacheManager(model.cache_specs(), num_pages=64, page_size=8, max_requests=4,
                         max_context=model.max_positions, dtype=dtype, device=model.device)
    cache.poison()
    runner = StepRunner(model, cache, max_step_tokens=16)
    requests = {"a": harness.random_tokens(cfg, 40, 1), "b": harness.random_tokens(cfg, 300, 2)}
    schedule = harness.tail_decode_schedule(requests, tail=8)      # a: 32 + 8 x 1, then b: 292 + 8 x 1
    actual = harness.run_schedule(runner, cache, schedule)
    assert runner._graphs, "single-token steps should have been recorded"
    expected = harness.plain_rows(requests, weights, cfg, torch.float32)
    yardstick = harness.plain_rows(requests, weights, cfg, dtype) if dtype == torch.bfloat16 else None
    harness.assert_rows_close(actual, expected, dtype, "after the buffers grew", yardstick)


def test_long_prompts_take_the_tensor_memory_kernels(folders, monkeypatch):
    """Heads of 128 and whole prompts of several hundred tokens: the step must go through the tcgen05
    product with the fused q/k/v tail, the tcgen05 gate/up product and the tcgen05 attention (the replay
    cases above check their results; this checks that it is those kernels that produced them)."""
    from qwen_inference_lab_b200.kernels import attention_tc, gemm_tc
    calls = {"qkv": 0, "gate_up": 0, "attention": 0}
    def counted(module, name, key):
        original = getattr(module, name)
        def wrapper(*args, **kwargs):
            calls[key] += 1
            return original(*args, **kwargs)
        monkeypatch.setattr(module, name, wrapper)
    counted(gemm_tc, "gemm_tc_qkv", "qkv")
    counted(gemm_tc, "gemm_tc", "gate_up")
    counted(attention_tc, "prefill", "attention")
    folder, weights, requests = folders["D"]
    _, cache, runner = harness.build_engine_parts(folder, torch.bfloat16, num_pages=80, page_size=16)
    harness.run_schedule(runner, cache, harness.whole_schedule(requests))      # ends with ``runner.check()``
    layers = TINY_D["num_hidden_layers"]
    lengths = [len(tokens) for tokens in requests.values()]
    assert calls["qkv"] == sum(n >= gemm_tc.QKV_TAIL_MIN_ROWS for n in lengths) * layers == 3 * layers
    assert calls["gate_up"] == len(lengths) * layers and calls["attention"] == len(lengths) * layers


def test_decoding_with_32_feature_blocks_in_the_products(folders, monkeypatch):
    """The decode product's form with two weight tiles a block is chosen by the width of the matrix, which no tiny
    configuration reaches: here every product whose width is a multiple of 32 is made to take it (q/k/v of tiny D with
    its bias and the norm inside, gate/up of tiny C with the activation behind, every product of tiny A down to the
    float32 head), in single-token steps against the plain rows."""
    from qwen_inference_lab_b200.kernels import ops, tuning
    monkeypatch.setattr(tuning, "SMALL_M_WIDE_MIN_BLOCKS", 1)
    taken = {16: 0, 32: 0}
    original = ops.core().qil_gemm_small_m
    def counted(*args):
        taken[args[12].value] += 1
        return original(*args)
    monkeypatch.setattr(ops.core(), "qil_gemm_small_m", counted)
    for case in ("D", "C", "A"):
        folder, weights, requests = folders[case]
        cfg, page_size = CASES[case]["cfg"], CASES[case]["page_size"]
        schedule = harness.tail_decode_schedule(requests, tail=12)
        num_pages = harness.peak_pages(schedule, page_size) + 1
        _, cache, runner = harness.build_engine_parts(folder, torch.bfloat16, num_pages=num_pages, page_size=page_size)
        actual = harness.run_schedule(runner, cache, schedule)
        expected = harness.plain_rows(requests, weights, cfg, torch.float32)
        yardstick = harness.plain_rows(requests, weights, cfg, torch.bfloat16)
        harness.assert_rows_close(actual, {k: expected[k] for k in actual}, torch.bfloat16, f"tiny {case}, wide blocks",
                                  {k: yardstick[k] for k in actual})
    assert taken[32] > 0 and taken[16] > 0
