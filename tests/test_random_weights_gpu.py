"""Random weights are a function of (seed, tensor name, element): the same bits wherever they are drawn."""
import pytest
import torch

from tests import harness
from tests.tiny_configs import TINY_B, TINY_D, typed

pytestmark = pytest.mark.gpu


def test_kernel_and_host_draw_the_same_bits():
    from qwen_inference_lab_b200.kernels import ops
    from qwen_inference_lab_b200.weights.random_init import normal_values
    for count, seed, std, mean, dtype in ((100003, 5, 0.02, 0.0, torch.bfloat16), (70001, 2**63 + 11, 0.05, 1.0, torch.float32),
                                          (4096, 0, 1.0, 0.0, torch.float32)):
        on_device = ops.fill_normal(torch.empty(count, dtype=dtype, device="cuda"), seed, std, mean).cpu()
        on_host = torch.from_numpy(normal_values(count, seed & (2**64 - 1), std, mean)).to(dtype)
        assert torch.equal(on_device, on_host)
    z = torch.from_numpy(normal_values(1 << 18, 99, 1.0))
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1) < 0.01 and 2.8 < (z ** 4).mean() < 3.1


@pytest.mark.parametrize("cfg,seed", [(TINY_B, 4), (TINY_D, 9)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_a_model_drawn_on_the_device_is_the_model_of_the_written_folder(tmp_path, cfg, seed, dtype):
    from qwen_inference_lab_b200 import Qwen3
    from qwen_inference_lab_b200.cache import CacheManager
    from qwen_inference_lab_b200.engine import StepEntry, StepRunner
    from qwen_inference_lab_b200.weights import SafetensorsFile, write_model_folder
    config = typed(cfg)
    drawn = Qwen3.random(config, seed, dtype=dtype)
    folder = write_model_folder(config, seed, tmp_path / "model", device="cpu",      # the host's draw against the device's
                                storage=torch.float32 if dtype == torch.float32 else torch.bfloat16)
    loaded = Qwen3.from_directory(folder, dtype=dtype)
    stacked_a, stacked_b = drawn.layers[-1].mixer.qkv._weight(), loaded.layers[-1].mixer.qkv._weight()
    assert stacked_a.dtype == dtype and torch.equal(stacked_a, stacked_b)
    assert torch.equal(drawn.final_norm.weight.data, loaded.final_norm.weight.data)
    assert torch.equal(drawn.embedding.weight.data, loaded.embedding.weight.data)
    with SafetensorsFile(folder / "model.safetensors") as f:
        assert torch.equal(f.tensor("model.embed_tokens.weight").cuda(), drawn.embedding.weight.data)
    tokens = harness.random_tokens(cfg, 50, 1)
    rows = []
    for model in (drawn, loaded):
        cache = CacheManager(model.cache_specs(), num_pages=8, page_size=16, max_requests=2,
                             max_context=model.max_positions, dtype=dtype, device=model.device)
        cache.admit("r")
        rows.append(StepRunner(model, cache).run([StepEntry("r", tokens, [49])]).cpu())
    assert torch.equal(rows[0], rows[1])
    # and the folder is an oracle for the drawn model: the plain implementation reads it
    with SafetensorsFile(folder / "model.safetensors") as f:
        weights = {name: f.tensor(name).float().clone() for name in f.keys()}      # the views die with the file
    if cfg.get("tie_word_embeddings", True):
        weights.setdefault("lm_head.weight", weights["model.embed_tokens.weight"])
    from tests.plain import qwen3_plain as plain
    expected = {("r", 49): plain.logits(tokens, weights, cfg)[49]}
    yardstick = {("r", 49): plain.logits(tokens, weights, cfg, dtype)[49]} if dtype == torch.bfloat16 else None
    if dtype == torch.float32:
        harness.assert_rows_close({("r", 49): rows[0][0]}, expected, dtype, "drawn model against the plain one")
    else:
        assert (rows[0][0] - expected[("r", 49)]).abs().max() < 4 * (yardstick[("r", 49)] - expected[("r", 49)]).abs().max()
