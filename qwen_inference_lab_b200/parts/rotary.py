"""Rotary position encoding as a table of cosines and sines.

``inv_freq[j] = 1 / theta^(2j / rotary_dim)`` and ``angle[p, j] = float(p) * inv_freq[j]``
are computed on the CPU in float32, as the reference does so that no device or
dtype conversion can round the frequencies (qil/model.py:99-108); cosine and sine
are then rounded to the activation dtype as in ``rotate`` (qil/model.py:42-46) and
kept as float32.  Mixers hand the table to their kernels: a kernel never derives
an angle itself, so another encoding (partial rotation, scaled frequencies) is
another table.
"""
from __future__ import annotations

import torch

from .base import PositionEncoding


def rotary_table(rotary_dim, theta, positions, dtype) -> torch.Tensor:
    """float32 [positions, rotary_dim]: cos of the rotary_dim/2 angles, then their sines."""
    exponent = torch.arange(0, rotary_dim, 2, device="cpu", dtype=torch.float32) / rotary_dim
    inv_freq = 1.0 / (theta ** exponent)
    angles = torch.arange(positions, device="cpu").float()[:, None] * inv_freq[None, :]
    table = torch.cat((angles.cos(), angles.sin()), dim=-1)
    return table.to(dtype).float().contiguous()


class RotaryEmbedding(PositionEncoding):
    graph_safe = True

    def __init__(self, rotary_dim, theta, max_positions):
        if rotary_dim % 2 or rotary_dim <= 0:
            raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
        self.rotary_dim, self.theta, self.max_positions = int(rotary_dim), float(theta), int(max_positions)
        self.table = None

    def finalize(self, device, dtype):
        self.table = rotary_table(self.rotary_dim, self.theta, self.max_positions, dtype).to(device)
