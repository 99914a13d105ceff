"""Typed model configuration, read from a checkpoint's own ``config.json`` keys.

Keys, defaults and rejections follow the reference's ``ModelConfig``
(qil/config.py:8-45): eight required positive integers, ``rms_norm_eps``,
``rope_theta``, ``attention_bias``, ``tie_word_embeddings`` and ``eos_token_id``
with the same defaults; ``model_type`` other than ``qwen3``, a ``rope_scaling``,
``use_sliding_window``, a ``layer_types`` entry other than ``full_attention`` and a
``hidden_act`` other than ``silu`` are refused.  No size lives in code: every part
of the model is built from these fields alone.
"""
from __future__ import annotations

from dataclasses import dataclass, fields
import json
import math
from pathlib import Path


class ConfigError(ValueError):
    """A config.json that this engine cannot run."""


_REQUIRED_INTS = (
    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings",
)


@dataclass(frozen=True)
class Qwen3Config:
    """Dense Qwen3 decoder (reference: qil/config.py:8-22)."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    attention_bias: bool = False
    tie_word_embeddings: bool = True
    eos_token_id: int | list | None = None

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    def __post_init__(self):
        for name in _REQUIRED_INTS:
            value = getattr(self, name)
            if type(value) is not int or value < 1:
                raise ConfigError(f"{name} must be a positive integer, got {value!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim must be even for half-split rotation, got {self.head_dim}")
        for name in ("rms_norm_eps", "rope_theta"):
            value = getattr(self, name)
            if isinstance(value, bool) or not isinstance(value, (int, float)) \
                    or not math.isfinite(value) or value <= 0:
                raise ConfigError(f"{name} must be positive and finite, got {value!r}")
        for name in ("attention_bias", "tie_word_embeddings"):
            if type(getattr(self, name)) is not bool:
                raise ConfigError(f"{name} must be a boolean")
        eos = self.eos_token_id
        if eos is not None:
            items = eos if isinstance(eos, list) else [eos]
            if any(type(t) is not int or t < 0 for t in items):
                raise ConfigError("eos_token_id must be an integer, a list of integers or null")

    @property
    def eos_token_ids(self) -> frozenset:
        eos = self.eos_token_id
        if eos is None:
            return frozenset()
        return frozenset(eos if isinstance(eos, list) else [eos])

    @classmethod
    def from_dict(cls, data: dict) -> "Qwen3Config":
        """Validate a parsed config.json (reference: qil/config.py:34-45)."""
        if data.get("model_type", cls.model_type) != cls.model_type:
            raise ConfigError(
                f"model_type {data.get('model_type')!r} is not the dense '{cls.model_type}' decoder")
        if data.get("rope_scaling") is not None:
            raise ConfigError("rope_scaling is not supported: only unscaled rotary positions")
        if data.get("use_sliding_window", False):
            raise ConfigError("use_sliding_window is not supported: every layer attends to all keys")
        if any(kind != "full_attention" for kind in data.get("layer_types") or []):
            raise ConfigError("layer_types must all be 'full_attention'")
        if data.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {data.get('hidden_act')!r} is not supported: only 'silu'")
        missing = [name for name in _REQUIRED_INTS if name not in data]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        known = {f.name for f in fields(cls)}
        return cls(**{key: data[key] for key in known if key in data})

    def to_dict(self) -> dict:
        data = {f.name: getattr(self, f.name) for f in fields(self)}
        data["architectures"] = [self.architecture]
        data["model_type"] = self.model_type
        data["hidden_act"] = "silu"
        return data


def read_config_json(directory) -> dict:
    path = Path(directory) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in {directory}")
    try:
        data = json.loads(path.read_text())
    except json.JSONDecodeError as error:
        raise ConfigError(f"{path} is not valid JSON: {error}") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return data
