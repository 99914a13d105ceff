"""Python face of the CUDA kernels: argument checks, then one C call per kernel.

Every function launches on torch's current CUDA stream and returns without
synchronising.  Tensors must live on the GPU and be contiguous; a wrong dtype,
shape or device raises before anything is launched.  There is no CPU path.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build, tuning

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

CORE_SOURCES = ["elementwise.cu", "rope_kv.cu", "gemm_f32.cu", "gemm_small_m.cu", "attention_generic.cu",
                "sampling.cu"]
SMALL_M_MAX_ROWS = min(16, tuning.SMALL_M_MAX_ROWS)      # the kernel takes 16 at most

_core = None


class KernelError(RuntimeError):
    pass


def core():
    global _core
    if _core is None:
        _core = build.load("qil_core", CORE_SOURCES)
    return _core


def dtype_code(dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


_post_step_checks: list = []


def register_post_step_check(check) -> None:
    """``check()`` raises if a kernel reported a fault of its own since the last call.  A kernel whose
    waits are bounded reports through an error word; its module registers the reader of that word here
    when its library is first loaded, and the step function's owner calls them after steps."""
    if check not in _post_step_checks:
        _post_step_checks.append(check)


def run_post_step_checks(wait=True) -> None:
    for check in _post_step_checks:
        check(wait)


class ErrorWord:
    """An int32 on the device that kernels with bounded waits set when a wait runs out, and its reader.

    ``check(wait=True)`` reads the word if a kernel that may set it was launched since the last check
    (``mark``); that waits for the device.  ``check(wait=False)`` never waits: it queues a copy of the
    word to pinned memory behind the work queued so far and reports what an earlier such copy
    brought, so a fault is reported a step or two late but the host never stalls a stream it is
    running ahead of.  The word stays set until it has been reported.
    """

    def __init__(self, describe):
        self._describe = describe
        self._word = self._host = self._event = None
        self._launched = self._copy_queued = False

    def tensor(self, device):
        if self._word is None:
            self._word = torch.zeros(1, dtype=torch.int32, device=device)
            self._host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
            self._event = torch.cuda.Event()
        return self._word

    def mark(self) -> None:
        self._launched = True

    def check(self, wait=True) -> None:
        if self._word is None:
            return
        code = 0
        if self._copy_queued and (wait or self._event.query()):
            self._event.synchronize()
            self._copy_queued = False
            code = int(self._host[0])
        if self._launched:
            self._launched = False
            if wait:
                code = code or int(self._word.item())
            else:
                self._host.copy_(self._word, non_blocking=True)
                self._event.record()
                self._copy_queued = True
        if code:
            self._word.zero_()
            self._copy_queued = False
            raise KernelError(self._describe(code))


_launches = 0


def launch_count() -> int:
    """Kernels launched through this module since import (graph replays are counted by their owner)."""
    return _launches


def _check(lib, code, what, kernels=1):
    global _launches
    if code != 0:
        raise KernelError(f"{what}: {lib.qil_last_error().decode()} (code {code})")
    _launches += kernels


def _p(tensor):
    return c_void_p(tensor.data_ptr()) if tensor is not None else c_void_p(0)


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(tensor, name, dtype=None, ndim=None):
    if not isinstance(tensor, torch.Tensor) or not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if ndim is not None and tensor.ndim != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got {tuple(tensor.shape)}")


def embed_gather(table, ids, out):
    """out[r] = table[ids[r]] cast to out's dtype.  table [V,H]; ids int32 [N]; out [N,H]."""
    _need(table, "table", ndim=2); _need(ids, "ids", torch.int32, 1); _need(out, "out", ndim=2)
    if out.shape != (ids.shape[0], table.shape[1]):
        raise KernelError(f"embed_gather: out {tuple(out.shape)} for ids {tuple(ids.shape)} table {tuple(table.shape)}")
    lib = core()
    _check(lib, lib.qil_embed_gather(_p(table), c_int(dtype_code(table.dtype)), _p(ids), _p(out),
                                     c_int(dtype_code(out.dtype)), c_int(ids.shape[0]), c_int(table.shape[1]),
                                     c_int(table.shape[0]), _stream()), "embed_gather")
    return out


def fill_normal(out, seed, std, mean=0.0):
    """out[i] = mean + std * z(seed, i), z close to N(0, 1) from a counter hash (the same bits as
    ``weights.random_init.normal_values`` gives on the host)."""
    _need(out, "out")
    lib = core()
    _check(lib, lib.qil_fill_normal(_p(out), c_int(dtype_code(out.dtype)), c_longlong(out.numel()),
                                    ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), c_float(std), c_float(mean),
                                    _stream()), "fill_normal")
    return out


def rmsnorm(x, weight, eps, out=None, rows=None):
    """RMSNorm over the last dimension; with ``rows`` (int32) only those rows, in that order."""
    _need(x, "x", ndim=2); _need(weight, "weight", ndim=1)
    width = x.shape[1]
    if weight.shape[0] != width:
        raise KernelError(f"rmsnorm: weight of {weight.shape[0]} for width {width}")
    n_rows = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
    if out is None:
        out = torch.empty((n_rows, width), dtype=x.dtype, device=x.device)
    _need(out, "out", x.dtype, 2)
    if out.shape != (n_rows, width):
        raise KernelError("rmsnorm: out has the wrong shape")
    lib = core()
    _check(lib, lib.qil_rmsnorm(_p(x), _p(weight), _p(rows), _p(out), c_int(n_rows), c_int(width),
                                c_float(eps), c_int(dtype_code(x.dtype)), c_int(dtype_code(weight.dtype)),
                                _stream()), "rmsnorm")
    return out


def silu_mul(gate_up, out=None, pairs8=False):
    """out = silu(gate) * up.  gate_up holds the gate columns then the up columns, or with
    ``pairs8`` groups of 16 columns: 8 gate columns followed by their 8 up columns."""
    _need(gate_up, "gate_up", ndim=2)
    if gate_up.shape[1] % 2:
        raise KernelError("silu_mul: the input's width must be even (gate columns then up columns)")
    width = gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((gate_up.shape[0], width), dtype=gate_up.dtype, device=gate_up.device)
    _need(out, "out", gate_up.dtype, 2)
    lib = core()
    _check(lib, lib.qil_silu_mul(_p(gate_up), _p(out), c_int(gate_up.shape[0]), c_int(width),
                                 c_int(dtype_code(gate_up.dtype)), c_int(1 if pairs8 else 0), _stream()), "silu_mul")
    return out


def small_m_ok(a, weight) -> bool:
    """Should ``gemm_small_m`` take this product?  bfloat16, at most 16 rows, K a multiple of 8.

    With 9 to 16 rows the kernel keeps three stages in flight instead of four; on a matrix as large
    as a vocabulary head (measured at 151936 x 4096: 274 us against the library's 211 us) that
    costs more than its epilogues save, so those go to the library.
    """
    if a.shape[0] > 8 and weight.shape[0] * weight.shape[1] >= tuning.SMALL_M_LIBRARY_ELEMENTS:
        return False
    return (a.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and a.shape[0] <= SMALL_M_MAX_ROWS
            and weight.shape[1] % 8 == 0 and a.is_contiguous())


def gemm_small_m(a, weight, bias=None, residual=None, out=None, out_float32=False, silu_pairs=False,
                 norm_weight=None, norm_eps=0.0, rows_per_block=None):
    """out = a @ weight.T (+ bias) (+ residual) for a decode step's few rows, streaming the weight once.

    a bfloat16 [M <= 16, K]; weight bfloat16 [N, K].  ``out_float32`` returns float32 (the LM head).
    ``silu_pairs``: weight rows are groups of [8 gate, 8 up]; returns silu(gate) * up, bfloat16 [M, N/2].
    ``residual`` may be ``out`` itself.  With ``norm_weight`` (bfloat16 [K]) the kernel first applies
    RMSNorm(a; norm_weight, norm_eps): the product of the normed rows, with no pass of its own over them.
    ``rows_per_block``: 16 or 32 output features a block (32 wants N a multiple of 32); None leaves it to the
    measured rule in ``tuning``.  The two forms add a product's terms in different orders.
    """
    _need(a, "a", torch.bfloat16, 2); _need(weight, "weight", torch.bfloat16, 2)
    m, k = a.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"gemm_small_m: a {tuple(a.shape)} against weight {tuple(weight.shape)}")
    out_shape = (m, n // 2) if silu_pairs else (m, n)
    out_dtype = torch.float32 if out_float32 else torch.bfloat16
    if bias is not None:
        _need(bias, "bias", torch.bfloat16, 1)
    if residual is not None:
        _need(residual, "residual", torch.bfloat16, 2)
        if residual.shape != out_shape:
            raise KernelError("gemm_small_m: residual has the wrong shape")
    if out is None:
        out = torch.empty(out_shape, dtype=out_dtype, device=a.device)
    _need(out, "out", out_dtype, 2)
    if out.shape != out_shape:
        raise KernelError("gemm_small_m: out has the wrong shape")
    if norm_weight is not None:
        _need(norm_weight, "norm_weight", torch.bfloat16, 1)
        if norm_weight.shape[0] != k:
            raise KernelError("gemm_small_m: the norm weight must have one value per input feature")
    if rows_per_block is None:
        wide = (n % 32 == 0 and n // 32 >= tuning.SMALL_M_WIDE_MIN_BLOCKS
                and (m > 8 or n * k < tuning.SMALL_M_WIDE_MAX_ELEMENTS))
        rows_per_block = 32 if wide else 16
    lib = core()
    _check(lib, lib.qil_gemm_small_m(_p(a), _p(weight), _p(bias), _p(residual), _p(out), _p(norm_weight),
                                     c_float(float(norm_eps)), c_int(m), c_int(n), c_int(k),
                                     c_int(1 if out_float32 else 0), c_int(1 if silu_pairs else 0),
                                     c_int(rows_per_block), _stream()),
           "gemm_small_m")
    return out


def feed_tokens(token_ids, pairs, count, source):
    """token_ids[pairs[2i]] = source[pairs[2i + 1]] for i < count, on the stream (all int32, on the device):
    fills the places of tokens that the previous step sampled and the host has not read yet."""
    _need(token_ids, "token_ids", torch.int32, 1); _need(pairs, "pairs", torch.int32, 1)
    _need(source, "source", torch.int32, 1)
    if pairs.shape[0] < 2 * count:
        raise KernelError("feed_tokens: fewer pairs than count")
    lib = core()
    _check(lib, lib.qil_feed_tokens(_p(token_ids), _p(pairs), c_int(count), _p(source), c_int(source.shape[0]),
                                    c_int(token_ids.shape[0]), _stream()), "feed_tokens")


def add_inplace(x, y):
    _need(x, "x"); _need(y, "y", x.dtype)
    if x.shape != y.shape:
        raise KernelError("add_inplace: shapes differ")
    lib = core()
    _check(lib, lib.qil_add_inplace(_p(x), _p(y), c_longlong(x.numel()), c_int(dtype_code(x.dtype)), _stream()),
           "add_inplace")
    return x


def cast(src, dtype, out=None):
    _need(src, "src")
    if out is None:
        out = torch.empty(src.shape, dtype=dtype, device=src.device)
    _need(out, "out", dtype)
    lib = core()
    _check(lib, lib.qil_cast(_p(src), c_int(dtype_code(src.dtype)), _p(out), c_int(dtype_code(dtype)),
                             c_longlong(src.numel()), _stream()), "cast")
    return out


def gemm_f32(a, weight, bias=None, residual=None, out=None):
    """out = a @ weight.T (+ bias) (+ residual), float32 accumulation on the CUDA cores.

    a [M,K] and out [M,N] share a dtype; weight [N,K] and bias [N] share another.
    ``residual`` may be ``out`` itself.
    """
    _need(a, "a", ndim=2); _need(weight, "weight", ndim=2)
    m, k = a.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"gemm_f32: a {tuple(a.shape)} against weight {tuple(weight.shape)}")
    if bias is not None:
        _need(bias, "bias", weight.dtype, 1)
        if bias.shape[0] != n:
            raise KernelError("gemm_f32: bias has the wrong length")
    if out is None:
        out = torch.empty((m, n), dtype=a.dtype, device=a.device)
    _need(out, "out", a.dtype, 2)
    if out.shape != (m, n):
        raise KernelError("gemm_f32: out has the wrong shape")
    if residual is not None:
        _need(residual, "residual", a.dtype, 2)
        if residual.shape != (m, n):
            raise KernelError("gemm_f32: residual has the wrong shape")
    lib = core()
    _check(lib, lib.qil_gemm_f32(_p(a), c_int(k), _p(weight), _p(bias), _p(residual), _p(out), c_int(m), c_int(n),
                                 c_int(k), c_int(dtype_code(a.dtype)), c_int(dtype_code(weight.dtype)), _stream()),
           "gemm_f32")
    return out


def qk_norm_rope_store(qkv, q_out, kv_cache, q_norm_w, k_norm_w, eps, rope_table, rotary_dim,
                       positions, token_row, block_table, n_q_heads, n_kv_heads, head_dim, page_size):
    """Norm and rotate q and k heads of ``qkv``, write q to ``q_out`` and k, v into ``kv_cache``.

    qkv [N, (Hq + 2*Hkv) * D]; q_out [N, Hq*D]; kv_cache [pages, 2, Hkv, P, D] (one layer);
    rope_table float32 [positions, rotary_dim] or None; block_table int32 [rows, max_pages].
    With n_kv_heads == 0 only queries are processed (a layer that reads another layer's cache).
    """
    _need(qkv, "qkv", ndim=2); _need(q_out, "q_out", qkv.dtype, 2)
    n = qkv.shape[0]
    if qkv.shape[1] != (n_q_heads + 2 * n_kv_heads) * head_dim or q_out.shape != (n, n_q_heads * head_dim):
        raise KernelError("qk_norm_rope_store: qkv/q_out shapes do not match the head counts")
    _need(positions, "positions", torch.int32, 1); _need(token_row, "token_row", torch.int32, 1)
    num_pages = 0
    if n_kv_heads:
        _need(kv_cache, "kv_cache", qkv.dtype, 5); _need(block_table, "block_table", torch.int32, 2)
        if tuple(kv_cache.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
            raise KernelError(f"qk_norm_rope_store: cache layout {tuple(kv_cache.shape)}")
        num_pages = kv_cache.shape[0]
    norm_code = F32
    if q_norm_w is not None:
        _need(q_norm_w, "q_norm_w", ndim=1); _need(k_norm_w, "k_norm_w", q_norm_w.dtype, 1)
        if q_norm_w.shape[0] != head_dim or k_norm_w.shape[0] != head_dim:
            raise KernelError("qk_norm_rope_store: norm weights must have head_dim elements")
        norm_code = dtype_code(q_norm_w.dtype)
    table_rows = 0
    if rope_table is not None:
        _need(rope_table, "rope_table", torch.float32, 2)
        if rope_table.shape[1] != rotary_dim:
            raise KernelError("qk_norm_rope_store: rope table width must equal rotary_dim")
        table_rows = rope_table.shape[0]
    lib = core()
    _check(lib, lib.qil_qk_norm_rope_store(
        _p(qkv), _p(q_out), _p(kv_cache if n_kv_heads else None), _p(q_norm_w), _p(k_norm_w), c_int(norm_code),
        c_float(eps), _p(rope_table), c_int(rotary_dim if rope_table is not None else 0), c_int(table_rows),
        _p(positions), _p(token_row), _p(block_table if n_kv_heads else None),
        c_int(block_table.shape[1] if n_kv_heads else 0), c_int(n), c_int(n_q_heads), c_int(n_kv_heads),
        c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(dtype_code(qkv.dtype)), _stream()),
        "qk_norm_rope_store")
    return q_out


def attention_generic(q, kv_cache, out, positions, token_row, block_table, n_q_heads, n_kv_heads,
                      head_dim, page_size, window, scale):
    """Causal GQA attention of every token over its request's pages (CUDA cores, float32 math)."""
    _need(q, "q", ndim=2); _need(out, "out", q.dtype, 2); _need(kv_cache, "kv_cache", q.dtype, 5)
    n = q.shape[0]
    if q.shape[1] != n_q_heads * head_dim or out.shape != q.shape:
        raise KernelError("attention_generic: q/out shapes do not match the head counts")
    if tuple(kv_cache.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
        raise KernelError(f"attention_generic: cache layout {tuple(kv_cache.shape)}")
    _need(positions, "positions", torch.int32, 1); _need(token_row, "token_row", torch.int32, 1)
    _need(block_table, "block_table", torch.int32, 2)
    lib = core()
    _check(lib, lib.qil_attention_generic(
        _p(q), _p(kv_cache), _p(out), _p(positions), _p(token_row), _p(block_table), c_int(block_table.shape[1]),
        c_int(n), c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size),
        c_int(kv_cache.shape[0]), c_int(window), c_float(scale), c_int(dtype_code(q.dtype)), _stream()),
        "attention_generic")
    return out


def sample_rows(logits, temperature=None, seed=None, counter=None, tokens=None, nonfinite=None, state=None,
                owner=None):
    """Choose one token per row of float32 ``logits`` [R,V]; returns (tokens, nonfinite) int32 [R].

    Settings per row come from arrays: temperature float32 [R] (0 = greedy), seed and counter int64 [R], all
    optional (greedy); or from state slots: ``state`` int64 [slots, 4] = (the temperature's float32 bits,
    seed, draws so far, unused) per request and ``owner`` int32 [R], the slot of each row.  With slots
    the kernel adds one to the draws of every row's slot.
    """
    _need(logits, "logits", torch.float32, 2)
    rows, vocab = logits.shape
    for name, t, dt in (("temperature", temperature, torch.float32), ("seed", seed, torch.int64),
                        ("counter", counter, torch.int64), ("owner", owner, torch.int32)):
        if t is not None:
            _need(t, name, dt, 1)
            if t.shape[0] != rows:
                raise KernelError(f"sample_rows: {name} needs one entry per row")
    if state is not None:
        _need(state, "state", torch.int64, 2)
        if state.shape[1] != 4 or owner is None:
            raise KernelError("sample_rows: state slots are int64 [slots, 4] and need the rows' owners")
    if tokens is None:
        tokens = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if nonfinite is None:
        nonfinite = torch.empty(rows, dtype=torch.int32, device=logits.device)
    lib = core()
    _check(lib, lib.qil_sample_rows(_p(logits), c_int(rows), c_int(vocab), c_longlong(logits.stride(0)),
                                    _p(temperature), _p(seed), _p(counter), _p(state), _p(owner), _p(tokens),
                                    _p(nonfinite), _stream()),
           "sample_rows")
    return tokens, nonfinite
