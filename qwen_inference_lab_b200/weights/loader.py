"""Strict loading of safetensors weights by tensor name.

Every ``*.safetensors`` file of the folder is read in sorted order, as the
reference does (qil/model.py:184-206); ``model.safetensors.index.json`` is not
needed.  Each tensor must be one the model expects, once, with the expected
shape; tied parameters that arrive under both names must be equal; every
expected parameter must be covered.  All problems of a folder are collected and
raised together as one :class:`WeightError`.

Storage: every floating-point tensor is cast to the run's dtype as it is loaded, as the
reference does (qil/model.py:197; tied tensors are compared after the cast), and integer
tables become int32.  In a bfloat16 run a tensor that the file stores in 32 bits stays
32-bit only where that is asked for: by its parameter (``Param.keep_32bit``, for
parameters whose part computes in float32) or for the whole folder with
``keep_stored_32bit=True`` (every product then runs on the slow 32-bit kernels).
``dtype=torch.float32`` (the true 32-bit path) widens everything to float32.
"""
from __future__ import annotations

from pathlib import Path

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """Missing, unexpected, duplicate, mis-shaped or inconsistent checkpoint tensors."""


def storage_dtype(stored: torch.dtype, run_dtype: torch.dtype, integer: bool, keep_32bit: bool = False) -> torch.dtype:
    if integer or not stored.is_floating_point:
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if keep_32bit and stored in (torch.float32, torch.float64):
        return torch.float32
    return run_dtype


def load_weights(model, directory, *, device, dtype, keep_stored_32bit=False) -> None:
    """Fill every Param of ``model`` from ``directory`` and finalize the model."""
    directory = Path(directory)
    expected = model.all_named_params()
    files = sorted(directory.glob("*.safetensors"))
    if not files:
        raise WeightError(f"no safetensors weights found in {directory}")
    unexpected, duplicate, wrong_shape, inconsistent, unreadable = [], [], [], [], []
    seen_names, mis_shaped = set(), set()
    for param in set(expected.values()):
        param.data = None
    for path in files:
        try:
            shard = SafetensorsFile(path)
        except SafetensorsError as error:
            unreadable.append(str(error))
            continue
        with shard:
            for name in shard.keys():
                param = expected.get(name)
                if param is None:
                    unexpected.append(name)
                    continue
                if name in seen_names:
                    duplicate.append(name)
                    continue
                seen_names.add(name)
                if tuple(shard.shape(name)) != param.shape:
                    wrong_shape.append(f"{name}: file has {list(shard.shape(name))}, model needs {list(param.shape)}")
                    mis_shaped.add(id(param))
                    continue
                source = shard.tensor(name)
                target = storage_dtype(source.dtype, dtype, param.integer, keep_stored_32bit or param.keep_32bit)
                value = source.to(device=device, dtype=target, copy=True)
                if param.data is not None:
                    # a second name of the same parameter (tied weights): values must agree
                    if param.data.dtype != value.dtype or not torch.equal(param.data, value):
                        inconsistent.append(name)
                    continue
                param.data = value
    # a tied parameter is satisfied by either of its names; a mis-shaped tensor is reported as such, not as missing
    missing = sorted(name for name, param in expected.items() if param.data is None and id(param) not in mis_shaped)
    problems = []
    if missing:
        problems.append(f"missing tensors ({len(missing)}): {missing}")
    if unexpected:
        problems.append(f"unexpected tensors ({len(unexpected)}): {sorted(unexpected)}")
    if duplicate:
        problems.append(f"tensors present more than once: {sorted(duplicate)}")
    if wrong_shape:
        problems.append("wrong shapes: " + "; ".join(wrong_shape))
    if inconsistent:
        problems.append(f"tied tensors with different values: {sorted(inconsistent)}")
    problems.extend(unreadable)
    if problems:
        raise WeightError(f"cannot load weights from {directory}: " + " | ".join(problems))
    model.finalize(device, dtype)
