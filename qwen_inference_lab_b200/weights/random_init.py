"""Random weights from a configuration and a seed.

Matrices and the embedding draw N(0, 0.02), norm weights 1 + N(0, 0.05), biases
zero.  Each tensor has its own generator seeded from (seed, tensor name), so the
values of one tensor do not depend on which other tensors exist.  The reference
ships no such mode; its tests draw a random model through another library
(tests/qil/conftest.py:11-25).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from ..config import registry
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def draw(param, seed, name, *, device="cpu", dtype=torch.bfloat16) -> torch.Tensor:
    generator = torch.Generator(device=device)
    generator.manual_seed(_tensor_seed(seed, name))
    if param.init == "zeros":
        return torch.zeros(param.shape, dtype=dtype, device=device)
    values = torch.randn(param.shape, generator=generator, dtype=torch.float32, device=device) * param.std
    if param.init == "norm":
        values += 1.0
    return values.to(dtype)


def random_state(model, seed, *, device="cpu", dtype=torch.bfloat16) -> dict:
    """Checkpoint name -> tensor; a tied parameter appears once, under its first name."""
    tensors, done = {}, set()
    for name, param in model.all_named_params().items():
        if id(param) in done:
            continue
        done.add(id(param))
        tensors[name] = draw(param, seed, name, device=device, dtype=dtype)
    return tensors


def init_random(model, seed, *, device, dtype, storage=None) -> None:
    """Fill ``model`` with random weights on ``device`` without going through a file."""
    storage = storage or (torch.float32 if dtype == torch.float32 else torch.bfloat16)
    done = set()
    for name, param in model.all_named_params().items():
        if id(param) in done:
            continue
        done.add(id(param))
        param.data = draw(param, seed, name, device=device, dtype=storage)
    model.finalize(device, dtype)


def write_model_folder(config, seed, directory, *, storage=torch.bfloat16) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed configuration)."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    data = config.to_dict()
    entry = registry.lookup(data)
    model = entry.build(config)
    (directory / "config.json").write_text(json.dumps(data, indent=2) + "\n")
    write_safetensors(directory / "model.safetensors", random_state(model, seed, dtype=storage),
                      metadata={"format": "pt", "seed": seed})
    return directory
