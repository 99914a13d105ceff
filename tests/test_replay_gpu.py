"""Replay of the same requests under four ways of cutting the work, against the plain implementation."""
import pytest
import torch

from tests import harness
from tests.tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D

pytestmark = pytest.mark.gpu

CASES = {
    "A": dict(cfg=TINY_A, seed=0, page_size=4, lengths=(5, 17, 33, 90)),
    "B": dict(cfg=TINY_B, seed=1, page_size=8, lengths=(1, 9, 31, 64, 100, 150)),
    "C": dict(cfg=TINY_C, seed=2, page_size=16, lengths=(40, 3, 130, 70)),
    "D": dict(cfg=TINY_D, seed=3, page_size=16, lengths=(700, 300, 1100)),
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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", list(SCHEDULES))
@pytest.mark.parametrize("case", list(CASES))
def test_replay_matches_plain(folders, case, schedule, dtype):
    folder, weights, requests = folders[case]
    cfg, page_size = CASES[case]["cfg"], CASES[case]["page_size"]
    longest = max(len(t) for t in requests.values())
    # so few pages that a mixed run must reuse the pages of finished requests
    live = 4 if schedule == "mixed" else 1
    num_pages = live * ((longest + page_size - 1) // page_size) if schedule == "mixed" \
        else (longest + page_size - 1) // page_size
    _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=num_pages, page_size=page_size)
    actual = harness.run_schedule(runner, cache, SCHEDULES[schedule](requests))
    assert cache.free_pages() == num_pages and not cache.owners()
    expected = harness.plain_rows(requests, weights, cfg, torch.float32)
    yardstick = harness.plain_rows(requests, weights, cfg, dtype) if dtype == torch.bfloat16 else None
    harness.assert_rows_close(actual, expected, dtype, f"tiny {case} {schedule} {dtype}", yardstick)


def test_recorded_steps_survive_a_step_that_outgrows_the_runner(folders):
    """Single-token steps are recorded as graphs; a later step with more tokens than the runner was
    made for replaces the buffers those graphs point into.  The recordings are then made anew, in a
    new memory pool, and the scratch that the parts keep between steps stays valid."""
    from qwen_inference_lab_b200.cache import CacheManager
    from qwen_inference_lab_b200.engine import StepRunner
    from qwen_inference_lab_b200.loading import load_model
    folder, weights, _ = folders["B"]
    cfg = CASES["B"]["cfg"]
    model = load_model(folder, device="cuda", dtype=torch.bfloat16)
    cache = CacheManager(model.cache_specs(), num_pages=64, page_size=8, max_requests=4,
                         max_context=model.max_positions, dtype=torch.bfloat16, device=model.device)
    cache.poison()
    runner = StepRunner(model, cache, max_step_tokens=16)
    requests = {"a": harness.random_tokens(cfg, 40, 1), "b": harness.random_tokens(cfg, 300, 2)}
    schedule = harness.tail_decode_schedule(requests, tail=8)      # a: 32 + 8 x 1, then b: 292 + 8 x 1
    actual = harness.run_schedule(runner, cache, schedule)
    assert runner._graphs, "single-token steps should have been recorded"
    expected = harness.plain_rows(requests, weights, cfg, torch.float32)
    yardstick = harness.plain_rows(requests, weights, cfg, torch.bfloat16)
    harness.assert_rows_close(actual, expected, torch.bfloat16, "after the buffers grew", yardstick)


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
    harness.run_schedule(runner, cache, harness.whole_schedule(requests))
    layers = TINY_D["num_hidden_layers"]
    assert calls["qkv"] == 2 * layers            # the prompts of 700 and 1100 tokens; 300 is below the tail's threshold
    assert calls["gate_up"] == 3 * layers and calls["attention"] == 3 * layers
    torch.cuda.synchronize()
    gemm_tc.check()
    attention_tc.check()
