"""Root-mean-square norm over the last dimension.

``y = cast(x32 * rsqrt(mean(x32^2) + eps)) * w``: statistics and scaling in float32,
rounded to the activation dtype, then multiplied by the weight (no ``1 + w``), as the
reference's ``ScaleNorm`` does (qil/model.py:15-23).
"""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, Param


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, width, eps, *, name):
        self.width, self.eps, self.name = int(width), float(eps), name
        self.weight = Param((width,), init="norm", std=0.05)

    def named_params(self):
        return {self.name + ".weight": self.weight}

    def forward(self, ctx, x, rows=None):
        """Norm of every row of ``x`` [N, width], or of ``x[rows]`` when ``rows`` (int32) is given."""
        return ops.rmsnorm(x, self.weight.data, self.eps, rows=rows)

    def as_rms(self):
        return self.weight.data, self.eps
