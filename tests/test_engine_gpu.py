"""Generation through the Python entry point, the scheduler's lifecycle on the GPU, long decoding."""
import json
import subprocess
import sys

import pytest
import torch

from tests import harness
from tests.plain import qwen3_plain as plain
from tests.tiny_configs import TINY_A, TINY_B, TINY_C

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    from qwen_inference_lab_b200 import Qwen3
    result = {}
    for name, cfg, seed in (("A", TINY_A, 0), ("B", TINY_B, 1), ("C", TINY_C, 2)):
        folder = tmp_path_factory.mktemp(f"tiny{name}")
        weights = harness.write_folder(cfg, seed, folder)
        result[name] = dict(folder=folder, weights=weights, cfg=cfg, loaded={})
    def get(name, dtype):
        entry = result[name]
        if dtype not in entry["loaded"]:
            entry["loaded"][dtype] = Qwen3.from_directory(entry["folder"], device="cuda", dtype=dtype)
        return entry["loaded"][dtype], entry["weights"], entry["cfg"]
    return get


check_greedy = harness.check_greedy


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("budget,chunk,pages,page_size", [(1, 1, 16, 4), (5, 3, 16, 8), (8, 8, 10, 8), (128, 64, 64, 4)])
def test_greedy_generation_matches_plain(models, dtype, budget, chunk, pages, page_size):
    from qwen_inference_lab_b200 import Engine
    model, weights, cfg = models("A", dtype)
    prompts = [harness.random_tokens(cfg, n, 70 + n) for n in (5, 17, 33)]
    engine = Engine(model, num_pages=pages, page_size=page_size, token_budget=budget, prefill_chunk=chunk,
                    max_active=4)
    rows = engine.generate(prompts, max_new_tokens=8, ignore_eos=True)
    for prompt, row in zip(prompts, rows):
        assert row["state"] == "completed" and row["finish_reason"] == "length" and len(row["token_ids"]) == 8
        check_greedy(prompt, row["token_ids"], weights, cfg, dtype)
    assert engine.idle and engine.cache.free_pages() == pages
    engine.cache.check_invariants()
    # steps made of single tokens are replayed from recorded graphs, cut into several pieces
    assert engine.runner.use_graphs and engine.runner._graphs
    assert all(len(record[0]) >= 1 for record in engine.runner._graphs.values())


def test_temperature_sampling_matches_plain_and_is_reproducible(models):
    from qwen_inference_lab_b200 import Engine
    model, weights, cfg = models("B", torch.float32)
    prompts = [harness.random_tokens(cfg, n, 90 + n) for n in (1, 9, 31, 64, 100)]
    def run(max_active, budget):
        engine = Engine(model, num_pages=64, page_size=8, prefill_chunk=16, token_budget=budget, max_active=max_active)
        return [row["token_ids"] for row in engine.generate(prompts, max_new_tokens=12, ignore_eos=True,
                                                            temperature=0.8, seed=4242)]
    first, second = run(4, 48), run(2, 17)
    assert first == second            # draws do not depend on batching
    greedy = Engine(model, num_pages=64, page_size=8).generate(prompts, max_new_tokens=12, ignore_eos=True)
    assert [row["token_ids"] for row in greedy] != first
    for index, (prompt, tokens) in enumerate(zip(prompts, first)):
        sequence = list(prompt)
        for counter, token in enumerate(tokens):
            logits = plain.logits(sequence, weights, cfg)[-1]
            assert token == plain.sample(logits, 0.8, 4242 + index, counter)
            sequence.append(token)


def test_sampling_settings_live_in_the_requests_slot_and_go_with_it(models):
    """A request's temperature, seed and draw count sit in its state slot on the device.  Requests that follow one
    another through the same two rows, some greedy, some sampling, with and without running a step ahead: each gets
    its own settings, a greedy one never inherits its predecessor's, and the draws are the plain implementation's."""
    from qwen_inference_lab_b200 import Engine
    model, weights, cfg = models("B", torch.float32)
    prompts = [harness.random_tokens(cfg, n, 300 + n) for n in (7, 12, 3, 20, 9, 5)]
    settings = [dict(temperature=0.9, seed=5), dict(), dict(temperature=0.0, seed=77), dict(temperature=1.4, seed=6),
                dict(), dict(temperature=0.9, seed=5)]
    for overlap in (False, True):
        engine = Engine(model, num_pages=48, page_size=8, token_budget=24, prefill_chunk=8, max_active=2, overlap=overlap)
        ids = [engine.submit(p, max_new_tokens=7, ignore_eos=True, **kw) for p, kw in zip(prompts, settings)]
        rows_used = {}
        while not engine.idle:
            engine.step()
            for rid in ids:
                if rid in engine.cache.rows:
                    rows_used.setdefault(rid, engine.cache.row(rid))
        assert sorted(set(rows_used.values())) == [0, 1] and len(rows_used) == 6      # six requests through two rows
        for rid, prompt, kw in zip(ids, prompts, settings):
            tokens = engine.result(rid)["token_ids"]
            sequence = list(prompt)
            for counter, token in enumerate(tokens):
                logits = plain.logits(sequence, weights, cfg)[-1]
                assert token == plain.sample(logits, kw.get("temperature", 0.0), kw.get("seed", 0), counter), \
                    f"request {rid} (overlap {overlap}) token {counter}"
                sequence.append(token)
        assert engine.cache.free_pages() == 48


def test_eos_cancel_arrival_and_failure(models, monkeypatch):
    from qwen_inference_lab_b200 import Engine
    model, weights, cfg = models("A", torch.float32)
    prompt = harness.random_tokens(cfg, 9, 3)
    greedy = plain.greedy(prompt, 6, weights, cfg)
    # the third generated token becomes an end-of-sequence token: it is emitted, then the request stops
    engine = Engine(model, num_pages=16, page_size=4)
    first = engine.submit(prompt, max_new_tokens=6)
    engine.scheduler.table[first].eos = {greedy[2]}
    second = None
    steps = 0
    while not engine.idle:
        engine.step()
        steps += 1
        if steps == 1:
            second = engine.submit(prompt[:4], max_new_tokens=3, ignore_eos=True)   # arrives between steps
    stop = greedy.index(greedy[2]) + 1
    assert engine.result(first)["token_ids"] == greedy[:stop] and engine.result(first)["finish_reason"] == "eos"
    assert engine.result(second)["token_ids"] == plain.greedy(prompt[:4], 3, weights, cfg)
    # cancelling an active and a waiting request frees everything
    engine = Engine(model, num_pages=16, page_size=4, max_active=1)
    a, b = engine.submit(prompt, max_new_tokens=5), engine.submit(prompt, max_new_tokens=5)
    engine.step()
    assert engine.cancel(a) and engine.cancel(b) and not engine.cancel(a)
    assert engine.idle and engine.cache.free_pages() == 16
    assert engine.result(a)["state"] == "cancelled" and engine.result(a)["e2e_s"] is None
    # a failing step retires its batch, frees its pages and leaves the waiting request runnable
    engine = Engine(model, num_pages=16, page_size=4, max_active=1)
    a, b = engine.submit(prompt, max_new_tokens=3), engine.submit(prompt[:5], max_new_tokens=3, ignore_eos=True)
    real_run = engine.runner.run
    monkeypatch.setattr(engine.runner, "run", lambda *args: (_ for _ in ()).throw(RuntimeError("injected")))
    with pytest.raises(RuntimeError, match="injected"):
        engine.step()
    assert engine.result(a)["state"] == "failed" and engine.result(a)["error"] == "injected"
    monkeypatch.setattr(engine.runner, "run", real_run)
    while not engine.idle:
        engine.step()
    assert engine.result(b)["token_ids"] == plain.greedy(prompt[:5], 3, weights, cfg)
    assert engine.cache.free_pages() == 16
    # non-finite logits are an error, not a token
    engine = Engine(model, num_pages=16, page_size=4)
    c = engine.submit(prompt, max_new_tokens=2)
    def broken(*args):
        engine.runner.logit_owner = torch.zeros(1, dtype=torch.int32, device="cuda")
        return torch.full((1, cfg["vocab_size"]), float("nan"), device="cuda")
    monkeypatch.setattr(engine.runner, "run", broken)
    with pytest.raises(RuntimeError, match="non-finite"):
        engine.step()
    assert engine.result(c)["state"] == "failed"


def test_running_a_step_ahead_gives_the_same_tokens(models, monkeypatch):
    """``overlap=True`` queues a step before the host has read the tokens of the step before it (they are fed
    on the device).  Same requests, same tokens, same reasons to stop as without; events come one call later;
    a request that stopped on an end-of-sequence token has one more token computed and dropped."""
    from qwen_inference_lab_b200 import Engine
    model, weights, cfg = models("B", torch.float32)
    prompts = [harness.random_tokens(cfg, n, 200 + n) for n in (5, 17, 33, 9, 2)]
    settings = [dict(max_new_tokens=10), dict(max_new_tokens=7, temperature=0.8, seed=11), dict(max_new_tokens=12),
                dict(max_new_tokens=1), dict(max_new_tokens=9)]
    greedy = plain.greedy(prompts[2], 12, weights, cfg)
    # the third request stops in mid-run, on a token that it has not generated before
    stop_at = max(k for k in range(1, 9) if greedy[k] not in greedy[:k])
    stop_token = greedy[stop_at]
    def run(overlap):
        engine = Engine(model, num_pages=40, page_size=8, token_budget=16, prefill_chunk=8, max_active=3,
                        overlap=overlap)
        ids, events, calls = [], [], 0
        for prompt, kw in zip(prompts[:4], settings[:4]):
            ids.append(engine.submit(prompt, ignore_eos=True, **kw))
        engine.scheduler.table[ids[2]].eos = {stop_token}
        while not engine.idle:
            got = engine.step()
            calls += 1
            if calls == 1:
                assert bool(got) != overlap or not got      # the first call of a run ahead has nothing to report yet
            if calls == 3:
                ids.append(engine.submit(prompts[4], ignore_eos=True, **settings[4]))     # arrives between steps
            events += [(e["request_id"], e["token_id"], e["finished"]) for e in got]
        assert engine.cache.free_pages() == 40 and not engine.cache.owners()
        engine.cache.check_invariants()
        return [engine.result(i) for i in ids], events, calls
    plain_rows, plain_events, plain_calls = run(False)
    ahead_rows, ahead_events, ahead_calls = run(True)
    for a, b in zip(plain_rows, ahead_rows):
        assert a["token_ids"] == b["token_ids"] and a["finish_reason"] == b["finish_reason"] and b["state"] == "completed"
    assert plain_rows[2]["finish_reason"] == "eos" and plain_rows[2]["token_ids"] == greedy[:stop_at + 1]
    assert plain_rows[3]["token_ids"] == plain.greedy(prompts[3], 1, weights, cfg)
    assert sorted(plain_events) == sorted(ahead_events)
    assert ahead_calls >= plain_calls
    # cancelling a request whose token is still on the device
    engine = Engine(model, num_pages=40, page_size=8, overlap=True)
    a = engine.submit(prompts[1], max_new_tokens=6, ignore_eos=True)
    engine.step(); engine.step(); engine.step()
    assert engine.cancel(a)
    assert engine.step() == [] and engine.idle and engine.cache.free_pages() == 40
    assert engine.result(a)["state"] == "cancelled"
    # a step that fails while the one before it is still unread: that one's tokens are kept, the batch is retired
    engine = Engine(model, num_pages=40, page_size=8, overlap=True, max_active=1)
    a, b = engine.submit(prompts[0], max_new_tokens=4, ignore_eos=True), engine.submit(prompts[3], max_new_tokens=2, ignore_eos=True)
    engine.step()
    real_run = engine.runner.run
    monkeypatch.setattr(engine.runner, "run", lambda *args: (_ for _ in ()).throw(RuntimeError("injected")))
    with pytest.raises(RuntimeError, match="injected"):
        engine.step()
    monkeypatch.setattr(engine.runner, "run", real_run)
    assert engine.result(a)["state"] == "failed" and engine.result(a)["token_ids"] == plain.greedy(prompts[0], 1, weights, cfg)
    while not engine.idle:
        engine.step()
    assert engine.result(b)["token_ids"] == plain.greedy(prompts[3], 2, weights, cfg)
    assert engine.cache.free_pages() == 40


def test_bad_submissions_are_rejected_without_allocation(models):
    from qwen_inference_lab_b200 import Engine
    model, _, cfg = models("A", torch.float32)
    engine = Engine(model, num_pages=4, page_size=4)
    for bad in ([], [-1], [cfg["vocab_size"]], [True], [1.0]):
        with pytest.raises(ValueError):
            engine.submit(bad)
    with pytest.raises(ValueError):
        engine.submit([1], max_new_tokens=0)
    with pytest.raises(ValueError):
        engine.submit([1] * 200, max_new_tokens=100)          # beyond max_position_embeddings
    with pytest.raises(ValueError):
        engine.submit([1] * 10, max_new_tokens=10)            # beyond the cache's 16 tokens
    with pytest.raises(ValueError):
        engine.submit([1], temperature=-1.0)
    assert engine.idle and engine.cache.free_pages() == 4 and not engine.cache.owners()
    with pytest.raises(ValueError):
        engine.generate([[1, 2], [1] * 30], max_new_tokens=4)  # the second cannot fit: the first is cleaned up
    assert engine.idle and engine.cache.free_pages() == 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(models, dtype):
    """300 tokens decoded one by one after a 3-token prompt (crosses the 256-position span of the
    single-token attention and many pages), every position's logits against the plain implementation."""
    model, weights, cfg = models("C", dtype)
    from qwen_inference_lab_b200.cache import CacheManager
    from qwen_inference_lab_b200.engine import StepRunner
    tokens = harness.random_tokens(cfg, 303, 21)
    cache = CacheManager(model.cache_specs(), num_pages=20, page_size=16, max_requests=2,
                         max_context=model.max_positions, dtype=dtype, device=model.device)
    cache.poison()
    runner = StepRunner(model, cache)
    schedule = [([("r", tokens[:1], [0])], []), ([("r", tokens[1:3], [0, 1])], [])]
    schedule += [([("r", tokens[i:i + 1], [0])], []) for i in range(3, len(tokens))]
    schedule[-1] = (schedule[-1][0], ["r"])
    actual = harness.run_schedule(runner, cache, schedule)
    requests = {"r": tokens}
    expected = harness.plain_rows(requests, weights, cfg, torch.float32)
    yardstick = harness.plain_rows(requests, weights, cfg, dtype) if dtype == torch.bfloat16 else None
    harness.assert_rows_close(actual, expected, dtype, f"long decode {dtype}", yardstick)


def test_command_line_generates(models, tmp_path):
    _, weights, cfg = models("A", torch.float32)
    folder = tmp_path / "model"
    harness.write_folder(cfg, 0, folder)
    prompt = harness.random_tokens(cfg, 7, 5)
    output = tmp_path / "out" / "result.json"
    done = subprocess.run([sys.executable, "-m", "qwen_inference_lab_b200", "--model", str(folder), "--token-ids",
                           json.dumps(prompt), "--dtype", "float32", "--max-new-tokens", "5", "--pages", "8",
                           "--page-size", "4", "--chunk-size", "3", "--ignore-eos", "--output", str(output)],
                          capture_output=True, text=True, cwd=str(harness.Path(__file__).resolve().parent.parent))
    assert done.returncode == 0, done.stderr
    result = json.loads(output.read_text())
    assert result == json.loads(done.stdout)
    assert result["token_ids"] == plain.greedy(prompt, 5, weights, cfg)
    assert result["state"] == "completed" and result["ttft_s"] is not None
