"""The host's plan for the single-token attention (no GPU): how many spans a context is cut into."""
from qwen_inference_lab_b200.kernels import attention_mma


def test_plans_cover_the_context_and_stay_within_the_kernels_limits():
    for n_decode, lo, hi in ((1, 8192, 8192), (8, 8193, 16384), (64, 8192, 8192), (1, 1, 100), (256, 40000, 40000),
                             (3, 1, 1), (2, 65537, 131072), (1, 1, 512)):
        n_spans, longest = attention_mma.plan_spans(n_decode, 32, 8, hi, 128, lo)
        assert n_spans >= 1 and longest % 64 == 0 and 64 <= longest <= attention_mma.MAX_DECODE_SPAN
        assert n_spans * longest >= hi                          # the spans cover the longest context
        assert (n_spans - 1) * longest < hi + 64 * n_spans      # and are not longer than that takes
        assert attention_mma.choose_span(n_decode, 32, 8, hi) % 64 == 0


def test_few_requests_get_more_spans_than_many_and_one_wave_is_preferred():
    slots = attention_mma._slots(128)
    assert attention_mma.plan_spans(1, 32, 8, 8192)[0] > attention_mma.plan_spans(16, 32, 8, 8192)[0]
    assert attention_mma.plan_spans(1, 32, 8, 1024)[0] <= 16
    n_spans, _ = attention_mma.plan_spans(8, 32, 8, 8192)
    assert slots // 2 < 8 * 8 * n_spans <= slots                # batch 8: one wave that fills most of the slots


def test_a_step_asks_every_layer_and_pays_once():
    attention_mma.plan_spans(5, 16, 8, 3000, 128)
    before = attention_mma._plan_tiles.cache_info()
    for _ in range(28):
        attention_mma.plan_spans(5, 16, 8, 3001, 128)           # the same tiles of context: remembered
    after = attention_mma._plan_tiles.cache_info()
    assert after.misses == before.misses and after.hits == before.hits + 28
