"""Gated feed-forward: ``down(silu(gate(x)) * up(x))`` (qil/model.py:38-40,70-71).

gate and up are one stacked product; the activation rounds ``silu(gate)`` to the
activation dtype before the multiply, as elementwise tensor code does.  In
bfloat16 the product and the activation are one kernel: the weight-streaming
kernel for a decode step's few rows, the tcgen05 kernel for prompt portions.
"""
from __future__ import annotations

import torch

from ..kernels import gemm_tc, ops
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

        self.pairs8 = False

    def children(self):
        return [self.gate_up, self.down]

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        w = self.gate_up._w
        inner = self.intermediate_size
        if w.dtype == torch.bfloat16 and inner % 8 == 0 and self.hidden_size % 8 == 0:
            # rows as groups of [8 gate, 8 up]: a block of the decode GEMM then holds matching gate and up
            # features and applies the activation in its epilogue
            self.gate_up._w = w.view(2, inner // 8, 8, self.hidden_size).transpose(0, 1).reshape(
                2 * inner, self.hidden_size).contiguous()
            self.pairs8 = True

    takes_norm = True

    def forward(self, ctx, x, residual=None, norm=None):
        """With ``norm`` x is the block's un-normed input; a decode step's few rows get the norm inside
        the gate/up kernel, longer steps a norm kernel of their own."""
        rms = norm.as_rms() if norm is not None else None
        if self.pairs8 and ops.small_m_ok(x, self.gate_up._w) and rms is not None and rms[0].dtype == torch.bfloat16:
            hidden = ops.gemm_small_m(x, self.gate_up._w, silu_pairs=True, norm_weight=rms[0], norm_eps=rms[1])
            return self.down.forward(ctx, hidden, residual=residual)
        if norm is not None:
            x = norm.forward(ctx, x)
        if self.pairs8 and ops.small_m_ok(x, self.gate_up._w):
            hidden = ops.gemm_small_m(x, self.gate_up._w, silu_pairs=True)
        elif self.pairs8 and gemm_tc.usable(x, self.gate_up._w):
            # prompt portions: the tcgen05 kernel applies the activation in its epilogue, so the
            # [tokens, 2 * intermediate] product never goes to memory
            hidden = gemm_tc.gemm_tc(x, self.gate_up._w, silu_pairs=True)
        else:
            gate_up = self.gate_up.forward(ctx, x)
            hidden = ops.silu_mul(gate_up, pairs8=self.pairs8)
        return self.down.forward(ctx, hidden, residual=residual)
