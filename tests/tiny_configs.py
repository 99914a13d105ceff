"""The small configurations the tests run: they differ in every size and option."""
import torch

from qwen_inference_lab_b200.config import Qwen3Config
import qwen_inference_lab_b200.models  # noqa: F401  (registers the architecture)
from qwen_inference_lab_b200.config import registry
from qwen_inference_lab_b200.weights import random_state

# tied embeddings, group of 2, head_dim 16, hidden == heads * head_dim
TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256, hidden_size=64,
              intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, max_position_embeddings=256, rope_theta=10000.0, rms_norm_eps=1e-6,
              attention_bias=False, tie_word_embeddings=True, eos_token_id=None)
# untied head, group of 3, head_dim 32, heads * head_dim != hidden, sizes that are no power of two
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1000, hidden_size=96,
              intermediate_size=200, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2,
              head_dim=32, max_position_embeddings=512, rope_theta=1000000.0, rms_norm_eps=1e-5,
              attention_bias=False, tie_word_embeddings=False, eos_token_id=[7, 9])
# biases on the attention projections, one kv head, head_dim 48, odd vocabulary
TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=517, hidden_size=80,
              intermediate_size=176, num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=1,
              head_dim=48, max_position_embeddings=640, rope_theta=50000.0, rms_norm_eps=3e-6,
              attention_bias=True, tie_word_embeddings=False, eos_token_id=3)

# heads of 128 and a width that the tcgen05 kernels take: long prompts of this one go through the
# tensor-memory product (pairs of SMs from 256 tokens on), its fused q/k/v tail (from 512 tokens on)
# and the tensor-memory attention (whole tiles of 128 tokens)
TINY_D = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1500, hidden_size=192,
              intermediate_size=328, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2,
              head_dim=128, max_position_embeddings=2048, rope_theta=1000000.0, rms_norm_eps=1e-6,
              attention_bias=True, tie_word_embeddings=True, eos_token_id=None)


def typed(cfg: dict) -> Qwen3Config:
    return Qwen3Config.from_dict(cfg)


def tiny_weights(cfg: dict, seed: int, dtype=torch.float32, bias_std=0.02) -> dict:
    """Checkpoint name -> CPU tensor for a tiny configuration (drawn by the engine's random mode).

    Values are drawn in bfloat16 so that both dtypes of a test see the same numbers;
    biases, which the random mode leaves at zero, get small random values here.
    """
    config = typed(cfg)
    model = registry.lookup(cfg).build(config)
    state = random_state(model, seed, dtype=torch.bfloat16)
    generator = torch.Generator().manual_seed(seed + 12345)
    for name in state:
        if name.endswith(".bias"):
            state[name] = (torch.randn(state[name].shape, generator=generator) * bias_std).to(torch.bfloat16)
    return {name: value.to(dtype) for name, value in state.items()}
