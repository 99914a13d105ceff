"""Dense Qwen3 as an arrangement of parts, with the checkpoint's tensor names.

Layer i is pre-norm: ``input_layernorm`` -> attention (q/k/v/o projections, per-head
``q_norm``/``k_norm``, rotary positions) -> residual -> ``post_attention_layernorm``
-> gated MLP (gate/up/down) -> residual; then ``model.norm`` and ``lm_head``, whose
weight is the embedding's when ``tie_word_embeddings`` (qil/model.py:26-40,89-98;
names as in ``checkpoint_parameters``, qil/model.py:159-176).
"""
from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.registry import register
from ..parts import (DecoderModel, GatedMLP, GroupedQueryAttention, LayerCall, Linear, PreNormBlock,
                     RMSNorm, RotaryEmbedding, TokenEmbedding)


def build_qwen3(config: Qwen3Config) -> DecoderModel:
    hidden = config.hidden_size
    rotary = RotaryEmbedding(config.head_dim, config.rope_theta, config.max_position_embeddings)
    layers = []
    for i in range(config.num_hidden_layers):
        prefix = f"model.layers.{i}."
        attention = GroupedQueryAttention(
            hidden, config.num_attention_heads, config.num_key_value_heads, config.head_dim,
            names={key: prefix + f"self_attn.{key}_proj" for key in "qkvo"}
            | {"q_norm": prefix + "self_attn.q_norm", "k_norm": prefix + "self_attn.k_norm"},
            bias=config.attention_bias, qk_norm_eps=config.rms_norm_eps, position=rotary)
        mlp = GatedMLP(hidden, config.intermediate_size,
                       names={key: prefix + f"mlp.{key}_proj" for key in ("gate", "up", "down")})
        layers.append(PreNormBlock(
            RMSNorm(hidden, config.rms_norm_eps, name=prefix + "input_layernorm"), attention,
            RMSNorm(hidden, config.rms_norm_eps, name=prefix + "post_attention_layernorm"), mlp))
    embedding = TokenEmbedding(config.vocab_size, hidden, name="model.embed_tokens")
    head = Linear(hidden, config.vocab_size, name="lm_head",
                  weight=embedding.weight if config.tie_word_embeddings else None)
    return DecoderModel(
        config=config, embedding=embedding, layers=layers,
        order=[LayerCall(i) for i in range(config.num_hidden_layers)],
        final_norm=RMSNorm(hidden, config.rms_norm_eps, name="model.norm"), head=head,
        max_positions=config.max_position_embeddings)


ARCHITECTURE = register(Qwen3Config.architecture, Qwen3Config.model_type, Qwen3Config, build_qwen3)
