"""Matrix products ``y = x W^T (+ b) (+ residual)`` with checkpoint-layout weights.

Weights are row-major ``[out_features, in_features]`` as the reference's
``nn.Linear`` stores them (qil/model.py:32-40).  A bfloat16 weight under bfloat16
activations goes to the library GEMM, which is what the reference's engine uses
for its projections (qil/model.py:52-54,69-71: ``nn.Linear`` -> cuBLAS); every
other combination (the true 32-bit path, or a weight stored in float32 inside a
bfloat16 model) runs the engine's own float32 CUDA-core product.  Products of at
most 16 rows (decode steps) run the engine's own weight-streaming kernel instead
of the library.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Param, Part


def _library_mm_f32_out(a, weight):
    """bf16 x bf16 -> float32 product without rounding the result to bfloat16."""
    try:
        return torch.mm(a, weight.t(), out_dtype=torch.float32)
    except TypeError:
        return torch.mm(a, weight.t()).float()


class Linear(Part):
    graph_safe = True

    def __init__(self, in_features, out_features, *, name, bias=False, weight=None):
        """``weight`` may be another part's Param of the same shape (tied embeddings)."""
        self.in_features, self.out_features = int(in_features), int(out_features)
        self.name = name
        if weight is not None and weight.shape != (self.out_features, self.in_features):
            raise ValueError(f"shared weight {weight.shape} does not fit [{out_features}, {in_features}]")
        self.weight = weight if weight is not None else Param((out_features, in_features))
        self.bias = Param((out_features,), init="zeros") if bias else None

    def named_params(self):
        params = {self.name + ".weight": self.weight}
        if self.bias is not None:
            params[self.name + ".bias"] = self.bias
        return params

    def finalize(self, device, dtype):
        if self.bias is not None and self.bias.data.dtype != self.weight.data.dtype:
            self.bias.data = self.bias.data.to(self.weight.data.dtype)   # the kernels read both as one dtype

    # The tensors the product runs with; StackedLinear overrides these.
    def _weight(self):
        return self.weight.data

    def _bias(self):
        return self.bias.data if self.bias is not None else None

    def forward(self, ctx, x, residual=None, out=None, out_float32=False, norm=None):
        """``x`` [N, in] -> [N, out]; adds ``residual`` [N, out] when given (may be ``out``).

        With ``norm`` (a Norm part) the product is of ``norm(x)``: fused into the kernel where it can be.
        """
        weight, bias = self._weight(), self._bias()
        if ops.small_m_ok(x, weight):
            # a decode step's few rows: the engine's weight-streaming kernel
            rms = norm.as_rms() if norm is not None else None
            if rms is not None and rms[0].dtype == torch.bfloat16:
                return ops.gemm_small_m(x, weight, bias=bias, residual=residual, out=out, out_float32=out_float32,
                                        norm_weight=rms[0], norm_eps=rms[1])
            if norm is not None:
                x = norm.forward(ctx, x)
            return ops.gemm_small_m(x, weight, bias=bias, residual=residual, out=out, out_float32=out_float32)
        if norm is not None:
            x = norm.forward(ctx, x)
        if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
            if out_float32:
                result = _library_mm_f32_out(x, weight)
                if bias is not None:
                    result += bias.float()
                return result
            if residual is not None and bias is None:
                return torch.addmm(residual, x, weight.t(), out=out if out is not None else residual)
            if bias is not None:
                result = torch.addmm(bias, x, weight.t(), out=out)
            else:
                result = torch.mm(x, weight.t(), out=out) if out is not None else torch.mm(x, weight.t())
            if residual is not None:
                ops.add_inplace(result, residual)
            return result
        # float32 accumulate on the CUDA cores; activations keep their dtype unless float32 is asked for
        if out_float32 and x.dtype != torch.float32:
            x = ops.cast(x, torch.float32)
        return ops.gemm_f32(x, weight, bias=bias, residual=residual, out=out)


class StackedLinear(Linear):
    """Several checkpoint matrices over the same input, run as one product.

    ``pieces`` is a list of (checkpoint name, out_features); the rows are stacked in
    that order after loading (the reference keeps q/k/v and gate/up apart,
    qil/model.py:32-34,38-39; one product over the stack reads the input once).
    """

    def __init__(self, in_features, pieces, *, bias=False):
        self.in_features = int(in_features)
        self.pieces = [(name, int(rows)) for name, rows in pieces]
        self.out_features = sum(rows for _, rows in self.pieces)
        self.parts_w = [Param((rows, in_features)) for _, rows in self.pieces]
        self.parts_b = [Param((rows,), init="zeros") for _, rows in self.pieces] if bias else None
        self._w = None
        self._b = None

    def named_params(self):
        params = {}
        for i, (name, _) in enumerate(self.pieces):
            params[name + ".weight"] = self.parts_w[i]
            if self.parts_b is not None:
                params[name + ".bias"] = self.parts_b[i]
        return params

    def finalize(self, device, dtype):
        dtypes = {p.data.dtype for p in self.parts_w}
        common = torch.float32 if len(dtypes) > 1 else dtypes.pop()
        self._w = torch.cat([p.data.to(common) for p in self.parts_w], dim=0).contiguous()
        for p in self.parts_w:
            p.data = None
        if self.parts_b is not None:
            self._b = torch.cat([p.data.to(common) for p in self.parts_b], dim=0).contiguous()
            for p in self.parts_b:
                p.data = None

    def _weight(self):
        return self._w

    def _bias(self):
        return self._b
