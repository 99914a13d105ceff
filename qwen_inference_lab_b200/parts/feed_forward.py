"""Gated feed-forward: ``down(silu(gate(x)) * up(x))`` (qil/model.py:38-40,70-71).

gate and up are one stacked product; the activation rounds ``silu(gate)`` to the
activation dtype before the multiply, as elementwise tensor code does.
"""
from __future__ import annotations

from ..kernels import ops
from .base import FeedForward
from .linear import Linear, StackedLinear


class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size, intermediate_size, *, names):
        """names: dict with keys gate, up, down (projection names without ``.weight``)."""
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.gate_up = StackedLinear(hidden_size, [(names["gate"], intermediate_size),
                                                   (names["up"], intermediate_size)])
        self.down = Linear(intermediate_size, hidden_size, name=names["down"])

    def children(self):
        return [self.gate_up, self.down]

    def forward(self, ctx, x, residual=None):
        gate_up = self.gate_up.forward(ctx, x)
        hidden = ops.silu_mul(gate_up)
        return self.down.forward(ctx, hidden, residual=residual)
