"""Compares the plain implementation with the reference's own model code, once.

Run on a machine that has the reference checkout:

    python tests/golden/make_golden.py /path/to/qwen-inference-lab

It draws the two tiny random models of the tests, loads the same tensors into the
reference's ``qil.model.Qwen3`` (through ``checkpoint_parameters``, qil/model.py:159-176)
on the CPU in float32, runs whole prompts through ``Qwen3.forward`` with a page pool
(qil/model.py:110-134) and the reference's ``Engine.generate`` (qil/engine.py:137-150),
checks the plain implementation against both, and stores tokens, logits and greedy
continuations in ``tests/golden/reference_outputs.pt`` for ``test_plain.py``.
"""
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests.plain import qwen3_plain as plain          # noqa: E402
from tests.tiny_configs import TINY_A, TINY_B, tiny_weights   # noqa: E402


def main(reference_root):
    sys.path.insert(0, str(reference_root))
    from qil.cache import PagePool
    from qil.config import ModelConfig
    from qil.engine import Engine
    from qil.model import Qwen3

    stored = {}
    for label, cfg, seed in (("A", TINY_A, 0), ("B", TINY_B, 1)):
        weights = tiny_weights(cfg, seed, torch.float32)
        fields = ModelConfig.__dataclass_fields__
        model = Qwen3(ModelConfig(**{k: v for k, v in cfg.items() if k in fields})).eval()
        with torch.no_grad():
            for name, parameter in model.checkpoint_parameters().items():
                source = name if name in weights else "model.embed_tokens.weight"
                parameter.copy_(weights[source])
        generator = torch.Generator().manual_seed(100 + seed)
        tokens = torch.randint(0, cfg["vocab_size"], (37,), generator=generator).tolist()
        pool = PagePool(layers=cfg["num_hidden_layers"], pages=16, page_size=4,
                        kv_heads=cfg["num_key_value_heads"], head_dim=cfg["head_dim"],
                        dtype=torch.float32, device="cpu")
        pool.admit("r", len(tokens))
        pool.ensure("r", len(tokens))
        reference_logits = model(tokens, start=0, pool=pool, request_id="r", logits_mode="all")
        ours = plain.logits(tokens, weights, cfg)
        difference = (ours - reference_logits).abs().max().item()
        print(f"tiny {label}: plain vs reference logits, max abs difference {difference:.3e}")
        assert difference < 2e-5, difference
        engine = Engine(model, num_pages=32, page_size=4)
        prompts = [tokens[:5], tokens[5:22]]
        generated = [row["token_ids"] for row in engine.generate(prompts, max_new_tokens=8, ignore_eos=True)]
        ours_generated = [plain.greedy(p, 8, weights, cfg) for p in prompts]
        assert generated == ours_generated, (generated, ours_generated)
        stored[label] = dict(tokens=tokens, logits=reference_logits.clone(), prompts=prompts, generated=generated)
    torch.save(stored, Path(__file__).with_name("reference_outputs.pt"))
    print("stored", Path(__file__).with_name("reference_outputs.pt"))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/qwen-inference-lab")
    main(Path(sys.argv[1]))
