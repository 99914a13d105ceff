"""The plain implementation itself (no GPU): against the reference's stored outputs and its own parts."""
from pathlib import Path

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.tiny_configs import TINY_A, TINY_B, TINY_C, tiny_weights

GOLDEN = Path(__file__).parent / "golden" / "reference_outputs.pt"


@pytest.mark.parametrize("label,cfg,seed", [("A", TINY_A, 0), ("B", TINY_B, 1)])
def test_plain_matches_the_reference_models_stored_outputs(label, cfg, seed):
    """tests/golden/make_golden.py ran the reference's qil.model.Qwen3 and qil.engine.Engine on the CPU."""
    stored = torch.load(GOLDEN)[label]
    weights = tiny_weights(cfg, seed, torch.float32)
    ours = plain.logits(stored["tokens"], weights, cfg)
    torch.testing.assert_close(ours, stored["logits"], atol=2e-6, rtol=2e-5)     # tests/qil/test_model.py:33
    for prompt, generated in zip(stored["prompts"], stored["generated"]):
        assert plain.greedy(prompt, len(generated), weights, cfg) == generated


def test_logits_of_a_prefix_do_not_depend_on_what_follows():
    weights = tiny_weights(TINY_C, 2, torch.float32)
    generator = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, TINY_C["vocab_size"], (40,), generator=generator).tolist()
    full = plain.logits(tokens, weights, TINY_C)
    torch.testing.assert_close(plain.logits(tokens[:13], weights, TINY_C), full[:13], atol=2e-6, rtol=2e-5)


def test_parts():
    x = torch.randn(5, 12)
    w = torch.rand(12) + 0.5
    expected = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w
    torch.testing.assert_close(plain.rms_norm(x, w, 1e-5), expected)
    # rotation by position 0 is the identity; rotation preserves the norm of each pair
    q = torch.randn(4, 3, 8)
    angles = plain.rotary_angles(torch.arange(4), 8, 10000.0)
    rotated = plain.rotate(q, angles)
    torch.testing.assert_close(rotated[0], q[0])
    torch.testing.assert_close(rotated.square().sum(-1), q.square().sum(-1))
    # attention: the first token attends only to itself; a window of 1 returns v
    k, v = torch.randn(4, 1, 8), torch.randn(4, 1, 8)
    out = plain.causal_attention(q, k, v, 8 ** -0.5)
    torch.testing.assert_close(out[0], v[0].expand(3, 8))
    torch.testing.assert_close(plain.causal_attention(q, k, v, 1.0, window=1), v.expand(4, 3, 8))
    # sampling: greedy at temperature 0, and the noise is a pure function of its three arguments
    row = torch.tensor([0.1, 2.0, -1.0])
    assert plain.sample(row, 0.0, 1, 0) == 1
    assert plain.gumbel_uniform(3, 4, 5) == plain.gumbel_uniform(3, 4, 5) != plain.gumbel_uniform(3, 5, 5)
    assert 0.0 < plain.gumbel_uniform(0, 0, 0) < 1.0
