"""From a model folder (or a configuration and a seed) to a model ready to step.

``load_model`` is the generic door: config.json names the architecture, the
registry supplies its configuration class and builder, the weights are loaded
strictly by name.  ``Qwen3`` keeps the reference's entry point
(``Qwen3.from_directory(path, device=, dtype=)``, qil/model.py:178-206) and adds
``Qwen3.random`` for seeded random weights.
"""
from __future__ import annotations

import torch

from . import models  # noqa: F401  (registers the architectures)
from .config import registry
from .config.model_config import ConfigError, Qwen3Config
from .weights import init_random, load_weights

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16,
           torch.float32: torch.float32, torch.bfloat16: torch.bfloat16}


def resolve_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be float32 or bfloat16, got {dtype!r}") from None


def require_gpu(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("this engine runs on a CUDA device only (its kernels have no CPU path)")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available")
    return device


def load_model(directory, *, device="cuda", dtype=torch.bfloat16, keep_stored_32bit=False):
    """``keep_stored_32bit``: in a bfloat16 run, leave tensors that the folder stores in 32 bits as they
    are instead of casting them (``weights.loader``)."""
    device, dtype = require_gpu(device), resolve_dtype(dtype)
    entry, config = registry.read_model_config(directory)
    model = entry.build(config)
    load_weights(model, directory, device=device, dtype=dtype, keep_stored_32bit=keep_stored_32bit)
    return model


def random_model(config, seed=0, *, device="cuda", dtype=torch.bfloat16):
    """A model with seeded random weights drawn directly on the device."""
    device, dtype = require_gpu(device), resolve_dtype(dtype)
    entry = registry.lookup(config.to_dict())
    model = entry.build(config)
    init_random(model, seed, device=device, dtype=dtype)
    return model


class Qwen3:
    """The reference's model entry point, kept by name (qil/model.py:89, :178)."""

    @staticmethod
    def from_directory(path, *, device="cuda", dtype=torch.bfloat16):
        entry, config = registry.read_model_config(path)
        if entry.config_class is not Qwen3Config:
            raise ConfigError(f"{path} holds a {entry.name}, not a dense Qwen3")
        return load_model(path, device=device, dtype=dtype)

    @staticmethod
    def random(config, seed=0, *, device="cuda", dtype=torch.bfloat16):
        return random_model(config, seed, device=device, dtype=dtype)
