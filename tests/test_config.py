"""Configuration and registry (no GPU)."""
import json

import pytest

import qwen_inference_lab_b200.models  # noqa: F401
from qwen_inference_lab_b200.config import ConfigError, Qwen3Config, registry
from tests.tiny_configs import TINY_A, TINY_B, TINY_C


def test_reads_the_architectures_own_keys(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_B, torch_dtype="bfloat16", unknown_key=5)))
    entry, config = registry.read_model_config(tmp_path)
    assert entry.name == "Qwen3ForCausalLM" and isinstance(config, Qwen3Config)
    for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "head_dim", "max_position_embeddings", "rms_norm_eps", "rope_theta",
                "attention_bias", "tie_word_embeddings"):
        assert getattr(config, key) == TINY_B[key]
    assert config.eos_token_ids == frozenset({7, 9})
    assert Qwen3Config.from_dict(config.to_dict()) == config


def test_defaults_follow_the_reference():
    minimal = {k: TINY_A[k] for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                      "num_attention_heads", "num_key_value_heads", "head_dim",
                                      "max_position_embeddings")}
    config = Qwen3Config.from_dict(dict(minimal, model_type="qwen3"))
    assert config.rms_norm_eps == 1e-6 and config.rope_theta == 1e6 and config.attention_bias is False
    assert config.tie_word_embeddings is True and config.eos_token_ids == frozenset()


@pytest.mark.parametrize("patch", [dict(model_type="qwen3_moe"), dict(rope_scaling={"rope_type": "linear"}),
                                   dict(use_sliding_window=True), dict(hidden_act="gelu"),
                                   dict(layer_types=["sliding_attention", "full_attention"]),
                                   dict(vocab_size=0), dict(hidden_size=-4), dict(num_hidden_layers=1.5),
                                   dict(num_attention_heads=5, num_key_value_heads=2), dict(head_dim=7),
                                   dict(rms_norm_eps=0.0), dict(rope_theta=float("inf")), dict(eos_token_id="x"),
                                   dict(tie_word_embeddings="yes")])
def test_unsupported_configurations_are_rejected(patch):
    with pytest.raises(ConfigError):
        Qwen3Config.from_dict(dict(TINY_A) | patch)


def test_missing_keys_and_files(tmp_path):
    broken = dict(TINY_A)
    del broken["head_dim"]          # the reference requires head_dim too: no hidden/heads fallback
    with pytest.raises(ConfigError, match="head_dim"):
        Qwen3Config.from_dict(broken)
    with pytest.raises(ConfigError):
        registry.read_model_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        registry.read_model_config(tmp_path)


def test_registry_maps_names_to_builders():
    assert "Qwen3ForCausalLM" in registry.known()
    assert registry.lookup({"architectures": ["Qwen3ForCausalLM"]}).config_class is Qwen3Config
    assert registry.lookup({"model_type": "qwen3"}).name == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        registry.lookup({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    with pytest.raises(ConfigError):
        registry.lookup({"model_type": "mystery"})
    with pytest.raises(ValueError):
        registry.register("Qwen3ForCausalLM", "qwen3", Qwen3Config, lambda config: None)


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_C])
def test_builder_takes_every_size_from_the_configuration(cfg):
    config = Qwen3Config.from_dict(cfg)
    model = registry.lookup(cfg).build(config)
    names = model.all_named_params()
    layers, d = cfg["num_hidden_layers"], cfg["head_dim"]
    per_layer = 11 + (4 if cfg["attention_bias"] else 0)
    assert len(names) == 3 + per_layer * layers
    assert (names["lm_head.weight"] is names["model.embed_tokens.weight"]) == cfg["tie_word_embeddings"]
    assert names["model.layers.0.self_attn.q_proj.weight"].shape == (cfg["num_attention_heads"] * d, cfg["hidden_size"])
    assert names["model.layers.0.self_attn.k_proj.weight"].shape == (cfg["num_key_value_heads"] * d, cfg["hidden_size"])
    assert names[f"model.layers.{layers - 1}.mlp.down_proj.weight"].shape == (cfg["hidden_size"], cfg["intermediate_size"])
    assert names["model.layers.0.self_attn.q_norm.weight"].shape == (d,)
    assert [call.layer for call in model.order] == list(range(layers))
    specs = model.cache_specs()
    assert all(s.kv_heads == cfg["num_key_value_heads"] and s.head_dim == d and s.window == 0 for s in specs)
    attention = model.layers[0].mixer
    assert attention.qk_norm_eps == cfg["rms_norm_eps"] and attention.position.theta == cfg["rope_theta"]
    assert attention.scale == d ** -0.5 and model.max_positions == cfg["max_position_embeddings"]
