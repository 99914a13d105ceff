"""Two layers at the sizes of a real checkpoint (hidden 4096, 32/8 heads of 128, 12288 wide, as Qwen3-8B) against the
plain implementation: the tiny configurations do not reach the kernel forms that the widths of a real model select
(32 output features a block in the decode products, the tile kernels' full tiles, spans over several waves of blocks)."""
import json

import pytest
import torch

from tests import harness
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

REAL = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=8192, hidden_size=4096,
            intermediate_size=12288, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8,
            head_dim=128, max_position_embeddings=1024, rope_theta=1000000.0, rms_norm_eps=1e-6,
            attention_bias=False, tie_word_embeddings=False, eos_token_id=None)


@pytest.fixture(scope="module")
def real_folder(tmp_path_factory):
    """The folder (weights drawn on the device, stored in bfloat16) and the same weights in float32 on the host."""
    from qwen_inference_lab_b200.config import registry
    from qwen_inference_lab_b200.weights import write_safetensors
    from qwen_inference_lab_b200.weights.random_init import random_state
    from tests.tiny_configs import typed
    folder = tmp_path_factory.mktemp("real_sizes")
    model = registry.lookup(REAL).build(typed(REAL))
    state = random_state(model, 11, device="cuda", dtype=torch.bfloat16)
    host = {name: tensor.cpu() for name, tensor in state.items()}
    (folder / "config.json").write_text(json.dumps(REAL))
    write_safetensors(folder / "model.safetensors", host)
    return folder, {name: tensor.float() for name, tensor in host.items()}


def test_two_real_layers_whole_prompts_then_single_tokens(real_folder, monkeypatch):
    from qwen_inference_lab_b200.kernels import ops
    folder, weights = real_folder
    requests = {"long": harness.random_tokens(REAL, 150, 3), "short": harness.random_tokens(REAL, 40, 4)}
    tail = 6
    # both prompts but their last ``tail`` tokens in one step, then one token each a step
    schedule = [([(rid, tokens[:-tail], [len(tokens) - tail - 1]) for rid, tokens in requests.items()], [])]
    for i in range(tail):
        schedule.append(([(rid, [tokens[len(tokens) - tail + i]], [0]) for rid, tokens in requests.items()],
                         list(requests) if i == tail - 1 else []))
    forms = {16: 0, 32: 0}
    original = ops.core().qil_gemm_small_m
    def counted(*args):
        forms[args[12].value] += 1
        return original(*args)
    monkeypatch.setattr(ops.core(), "qil_gemm_small_m", counted)
    wanted = {(rid, position) for rid, tokens in requests.items() for position in range(len(tokens) - tail - 1, len(tokens))}
    expected = {k: v for k, v in harness.plain_rows(requests, weights, REAL, torch.float32).items() if k in wanted}
    yardstick = {k: v for k, v in harness.plain_rows(requests, weights, REAL, torch.bfloat16).items() if k in wanted}
    for dtype in (torch.bfloat16, torch.float32):
        _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=16, page_size=16)
        actual = harness.run_schedule(runner, cache, schedule)
        if dtype == torch.bfloat16:
            harness.assert_rows_close(actual, expected, dtype, f"two real layers, {dtype}", yardstick)
        else:
            # Sums of 12288 float32 terms: the engine adds them in ascending k with one accumulator, the plain
            # implementation's library in blocks, and both are a random walk of roundings away from the exact sum:
            # about sqrt(K) * 2^-24 of the terms' size per product.  The bar allows 64 such steps on the way to a
            # logit (two layers of four products, the norms, the head), relative to the largest logit.
            assert set(actual) == set(expected)
            scale = max(float(row.abs().max()) for row in expected.values())
            bar = 64 * (REAL["intermediate_size"] ** 0.5) * 2.0 ** -24 * scale
            worst = max(expected, key=lambda k: float((actual[k] - expected[k]).abs().max()))
            error = float((actual[worst] - expected[worst]).abs().max())
            assert error <= bar, f"float32 logits differ by {error:.3e} at {worst} (bar {bar:.3e}, largest logit {scale:.3f})"
            for key, row in expected.items():
                best = row.topk(2).values
                if float(best[0] - best[1]) > 4 * bar:
                    assert int(actual[key].argmax()) == int(row.argmax()), f"another best token at {key}"
        del runner, cache
        torch.cuda.empty_cache()
    assert forms[32] > 0 and forms[16] > 0      # q/k/v and gate/up took the wide form, o and down the other (later steps replay)


def test_two_real_layers_long_prompts(real_folder):
    """Prompts long enough for the tensor-memory kernels at real head counts (the q/k/v product with its fused tail
    from 512 rows on, the paired gate/up product, whole 128-token attention tiles and what they leave over), whole and
    cut after 384 tokens, against the plain rows at a few positions."""
    folder, weights = real_folder
    requests = {"a": harness.random_tokens(REAL, 640, 5), "b": harness.random_tokens(REAL, 530, 6)}
    wants = {"a": [0, 127, 128, 400, 639], "b": [1, 255, 256, 511, 529]}
    whole = [([(rid, tokens, wants[rid])], [rid]) for rid, tokens in requests.items()]
    cut = [([("a", requests["a"][:384], [0, 127, 128]), ("b", requests["b"][:2], [1])], []),
           ([("a", requests["a"][384:], [400 - 384, 639 - 384]), ("b", requests["b"][2:], [253, 254, 509, 527])], ["a", "b"])]
    wanted = {(rid, position) for rid in requests for position in wants[rid]}
    expected = {k: v for k, v in harness.plain_rows(requests, weights, REAL, torch.float32).items() if k in wanted}
    yardstick = {k: v for k, v in harness.plain_rows(requests, weights, REAL, torch.bfloat16).items() if k in wanted}
    for name, schedule in (("whole", whole), ("cut", cut)):
        _, cache, runner = harness.build_engine_parts(folder, torch.bfloat16, num_pages=80, page_size=16)
        actual = harness.run_schedule(runner, cache, schedule)
        harness.assert_rows_close(actual, expected, torch.bfloat16, f"two real layers, long prompts, {name}", yardstick)
        del runner, cache
        torch.cuda.empty_cache()


def test_two_real_layers_sixty_four_requests_decoding_together(real_folder):
    """64 short requests that decode side by side: products of 64 rows (the library's and the tile kernel's), the
    single-token attention with a merge kernel behind it (a span's worth of blocks fills the GPU), recorded graphs."""
    folder, weights = real_folder
    requests = {f"r{i}": harness.random_tokens(REAL, 12 + (i * 7) % 19, 100 + i) for i in range(64)}
    tail = 3
    schedule = [([(rid, tokens[:-tail], []) for rid, tokens in requests.items()], [])]
    for i in range(tail):
        schedule.append(([(rid, [tokens[len(tokens) - tail + i]], [0]) for rid, tokens in requests.items()],
                         list(requests) if i == tail - 1 else []))
    wanted = {(rid, position) for rid, tokens in requests.items() for position in range(len(tokens) - tail, len(tokens))}
    expected = {k: v for k, v in harness.plain_rows(requests, weights, REAL, torch.float32).items() if k in wanted}
    yardstick = {k: v for k, v in harness.plain_rows(requests, weights, REAL, torch.bfloat16).items() if k in wanted}
    _, cache, runner = harness.build_engine_parts(folder, torch.bfloat16, num_pages=200, page_size=16, max_requests=64)
    actual = harness.run_schedule(runner, cache, schedule)
    assert runner._graphs, "the single-token steps should have been recorded"
    harness.assert_rows_close(actual, expected, torch.bfloat16, "two real layers, 64 requests", yardstick)
