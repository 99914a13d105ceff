"""Random weights from a configuration and a seed.

Matrices and the embedding draw N(0, 0.02), norm weights 1 + N(0, 0.05), biases
zero.  A value depends on (seed, tensor name, element index) alone: not on which
other tensors exist, and not on where it is drawn.  The host draws with numpy, the
GPU with a kernel (``ops.fill_normal``), and both give the same bits, so a model
drawn on the device, a model folder written on the host and the plain
implementation that reads that folder all hold the same weights.

The normal variate is the sum of twelve 16-bit uniforms from a 64-bit counter hash,
centred and scaled (mean 0, variance 1 - 2**-32, support +-6): integers and three
correctly rounded float32 operations, which is what makes host and device agree to
the bit.  The reference ships no such mode; its tests draw a random model through
another library (tests/qil/conftest.py:11-25).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np
import torch

from ..config import registry
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


_GOLDEN, _MIX1, _MIX2 = (np.uint64(v) for v in (0x9E3779B97F4A7C15, 0xBF58476D1CE4E5B9, 0x94D049BB133111EB))


def _hash(seed, counters):
    """splitmix64's output function over ``seed + (counter + 1) * golden`` (numpy uint64, wrapping)."""
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + (counters + np.uint64(1)) * _GOLDEN
        z ^= z >> np.uint64(30); z *= _MIX1
        z ^= z >> np.uint64(27); z *= _MIX2
        z ^= z >> np.uint64(31)
    return z


def normal_values(count, seed, std, mean=0.0, first=0) -> np.ndarray:
    """float32 [count]: elements ``first .. first + count`` of the stream of ``seed`` (host twin of
    ``fill_normal_kernel`` in csrc/elementwise.cu)."""
    index = np.arange(first, first + count, dtype=np.uint64)
    total = np.zeros(count, dtype=np.int64)
    mask = np.uint64(0xFFFF)
    for round_ in range(3):
        h = _hash(seed, np.uint64(3) * index + np.uint64(round_))
        for shift in (0, 16, 32, 48):
            total += ((h >> np.uint64(shift)) & mask).astype(np.int64)
    z = (total - 393210).astype(np.float32) * np.float32(1.0 / 65536.0)
    return z * np.float32(std) + np.float32(mean)


def draw(param, seed, name, *, device="cpu", dtype=torch.bfloat16) -> torch.Tensor:
    """The tensor of ``param`` under its checkpoint name ``name``: drawn where it is wanted."""
    device = torch.device(device)
    if param.init == "zeros":
        return torch.zeros(param.shape, dtype=dtype, device=device)
    mean = 1.0 if param.init == "norm" else 0.0
    stream_seed = _tensor_seed(seed, name)
    if device.type == "cuda":
        from ..kernels import ops
        return ops.fill_normal(torch.empty(param.shape, dtype=dtype, device=device), stream_seed, param.std, mean)
    count = 1
    for n in param.shape:
        count *= n
    out = torch.empty(count, dtype=dtype)
    step = 1 << 22                      # in pieces: the intermediates of a piece are 8 bytes an element
    for first in range(0, count, step):
        piece = normal_values(min(step, count - first), stream_seed, param.std, mean, first)
        out[first:first + len(piece)] = torch.from_numpy(piece).to(dtype)
    return out.reshape(param.shape)


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


def write_model_folder(config, seed, directory, *, storage=torch.bfloat16, device=None) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed configuration).

    The values are the same bits wherever they are drawn, so they are drawn on the GPU when there is one
    (``device=None``) and brought back tensor by tensor: a model of a billion parameters takes the host a minute."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    data = config.to_dict()
    entry = registry.lookup(data)
    model = entry.build(config)
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    tensors, done = {}, set()
    for name, param in model.all_named_params().items():
        if id(param) not in done:
            done.add(id(param))
            tensors[name] = draw(param, seed, name, device=device, dtype=storage).cpu()
    (directory / "config.json").write_text(json.dumps(data, indent=2) + "\n")
    write_safetensors(directory / "model.safetensors", tensors, metadata={"format": "pt", "seed": seed})
    return directory
