"""The tcgen05/TMA matrix product for prompt portions (bfloat16, float32 accumulation in tensor memory).

``gemm_tc(a, w, ...)`` computes ``a @ w.T`` with the epilogues of :func:`ops.gemm_small_m`.  The
kernel's mbarrier waits are bounded; if one runs out the kernel records where in an error word and
returns.  ``check()`` reads that word (it synchronises) and raises if it is set.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from . import build
from . import ops, tuning
from .ops import KernelError, _check, _need, _p, _stream

_lib = None
_sm_count = None
MIN_ROWS = tuning.TILE_KERNEL_MIN_ROWS


def _describe_fault(code):
    where = {1: "producer waiting for a free stage", 2: "producer draining its copies",
             3: "MMA issuer waiting for a free accumulator", 4: "MMA issuer waiting for a stage's data",
             5: "epilogue waiting for the accumulator"}.get(code, "unknown place")
    return f"gemm_tc: a wait inside the kernel ran out ({where}, code {code})"


_fault = ops.ErrorWord(_describe_fault)


def library():
    global _lib
    if _lib is None:
        _lib = build.load("qil_gemm_tc", ["gemm_tc.cu"])
        ops.register_post_step_check(check)
    return _lib


def error_word(device):
    """The kernels' error word, marked as possibly written: call right before a launch."""
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(device).multi_processor_count
    _fault.mark()
    return _fault.tensor(device)


def usable(a, weight) -> bool:
    """bfloat16 operands, enough rows to fill a tile's worth of work, 16-byte rows."""
    return (a.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and a.shape[0] >= MIN_ROWS
            and weight.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0 and a.is_contiguous())


def gemm_tc(a, weight, bias=None, residual=None, out=None, silu_pairs=False):
    """out = a @ weight.T (+ bias) (+ residual); with ``silu_pairs`` (weight rows as [8 gate, 8 up] groups)
    out = silu(gate) * up of width N/2.  ``residual`` may be ``out``."""
    _need(a, "a", torch.bfloat16, 2); _need(weight, "weight", torch.bfloat16, 2)
    m, k = a.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"gemm_tc: a {tuple(a.shape)} against weight {tuple(weight.shape)}")
    out_shape = (m, n // 2) if silu_pairs else (m, n)
    if bias is not None:
        _need(bias, "bias", torch.bfloat16, 1)
    if residual is not None:
        _need(residual, "residual", torch.bfloat16, 2)
        if residual.shape != out_shape:
            raise KernelError("gemm_tc: residual has the wrong shape")
    if out is None:
        out = torch.empty(out_shape, dtype=torch.bfloat16, device=a.device)
    _need(out, "out", torch.bfloat16, 2)
    if out.shape != out_shape:
        raise KernelError("gemm_tc: out has the wrong shape")
    word = error_word(a.device)
    lib = library()
    _check(lib, lib.qil_gemm_tc(_p(a), _p(weight), _p(bias), _p(residual), _p(out), c_int(m), c_int(n), c_int(k),
                                c_int(1 if silu_pairs else 0), c_int(_sm_count), _p(word), _stream()), "gemm_tc")
    return out


QKV_TAIL_MIN_ROWS = tuning.QKV_TAIL_MIN_ROWS


def qkv_tail_usable(a, weight, head_dim, rotary_dim, norm_weights, pages) -> bool:
    """Can ``gemm_tc_qkv`` take this projection?  Heads of 128, rotation of the whole head or none,
    bfloat16 everywhere, enough rows."""
    return (usable(a, weight) and a.shape[0] >= QKV_TAIL_MIN_ROWS and head_dim == 128 and rotary_dim in (0, 128)
            and all(w is None or w.dtype == torch.bfloat16 for w in norm_weights)
            and (pages is None or pages.dtype == torch.bfloat16))


def gemm_tc_qkv(a, weight, bias, q_out, pages, rope_table, q_norm, k_norm, eps, positions, token_row, block_table,
                n_q_heads, n_kv_heads, page_size):
    """The stacked q/k/v projection with its tail in the epilogue: per-head RMSNorm of queries and keys,
    rotation by position, queries into ``q_out`` [M, n_q_heads * 128], keys and values into the tokens'
    pages.  ``weight`` [(n_q_heads + 2 n_kv_heads) * 128, K]; ``n_kv_heads`` 0 for a layer without
    keys and values of its own; ``rope_table`` float32 [positions, 128] or None."""
    _need(a, "a", torch.bfloat16, 2); _need(weight, "weight", torch.bfloat16, 2)
    m, k = a.shape
    if weight.shape != ((n_q_heads + 2 * n_kv_heads) * 128, k):
        raise KernelError(f"gemm_tc_qkv: weight {tuple(weight.shape)} for {n_q_heads}+2x{n_kv_heads} heads of 128, K {k}")
    _need(q_out, "q_out", torch.bfloat16, 2)
    if q_out.shape != (m, n_q_heads * 128):
        raise KernelError("gemm_tc_qkv: q_out has the wrong shape")
    _need(positions, "positions", torch.int32, 1)
    if bias is not None:
        _need(bias, "bias", torch.bfloat16, 1)
    for name, w in (("q_norm", q_norm), ("k_norm", k_norm)):
        if w is not None:
            _need(w, name, torch.bfloat16, 1)
            if w.shape[0] != 128:
                raise KernelError(f"gemm_tc_qkv: {name} must have 128 values")
    num_pages = 0
    if n_kv_heads:
        _need(pages, "pages", torch.bfloat16); _need(token_row, "token_row", torch.int32, 1)
        _need(block_table, "block_table", torch.int32, 2)
        if tuple(pages.shape[1:]) != (2, n_kv_heads, page_size, 128):
            raise KernelError(f"gemm_tc_qkv: cache layout {tuple(pages.shape)}")
        num_pages = pages.shape[0]
    if rope_table is not None:
        _need(rope_table, "rope_table", torch.float32, 2)
        if rope_table.shape[1] != 128:
            raise KernelError("gemm_tc_qkv: the rotation must cover the whole head")
    word = error_word(a.device)
    lib = library()
    _check(lib, lib.qil_gemm_tc_qkv(
        _p(a), _p(weight), _p(bias), _p(q_out), _p(pages), _p(rope_table),
        c_int(rope_table.shape[0] if rope_table is not None else 0), _p(q_norm), _p(k_norm), c_float(float(eps)),
        _p(positions), _p(token_row), _p(block_table), c_int(block_table.shape[1] if block_table is not None else 0),
        c_int(n_q_heads), c_int(n_kv_heads), c_int(page_size), c_int(num_pages), c_int(m), c_int(k),
        c_int(_sm_count), _p(word), _stream()), "gemm_tc_qkv")
    return q_out


def check(wait=True) -> None:
    """Raise if a bounded wait inside a gemm_tc launch ran out (see ``ops.ErrorWord.check``)."""
    _fault.check(wait)
