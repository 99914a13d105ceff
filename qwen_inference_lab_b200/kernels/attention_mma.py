"""Tensor-core attention for bfloat16, compiled per head size on first use.

``attend`` runs both forms over one step's batch: query tiles of prompt portions
go to the tiled kernel, single tokens to the span kernel plus its merge.  The
span kernel's partial sums live in scratch that is allocated once per step and
shared by all layers.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from . import attention_tc, build
from .ops import KernelError, _check, _p, _stream

_libs: dict = {}
KV_TILE = 64
MAX_DECODE_SPAN = 2048


def supports(head_dim, n_q_heads, n_kv_heads) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256 and n_q_heads % n_kv_heads == 0


def library(head_dim):
    lib = _libs.get(head_dim)
    if lib is None:
        if not supports(head_dim, 1, 1):
            raise KernelError(f"the tensor-core attention takes head sizes 16, 32, ..., 256, not {head_dim}")
        lib = build.load(f"qil_attn_d{head_dim}", ["attention_mma.cu"], {"QIL_HEAD_DIM": head_dim})
        if lib.qil_attn_head_dim() != head_dim or lib.qil_attn_max_decode_span() != MAX_DECODE_SPAN:
            raise KernelError("attention library was built for other constants")
        _libs[head_dim] = lib
    return lib


_sm_count = None


def _slots(head_dim) -> int:
    """Blocks of the span kernel that run at a time: SMs x blocks per SM (shared memory decides)."""
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count \
            if torch.cuda.is_available() else 148
    block_smem = (16 + 4 * KV_TILE) * (head_dim + 8) * 2 + 2048
    return _sm_count * max(1, min(3, (227 * 1024) // block_smem))


def choose_span(n_decode, n_q_heads, n_kv_heads, max_context, head_dim=128) -> int:
    """Positions per block of the single-token kernel, from a small cost model.

    Blocks run in waves of (SMs x blocks per SM); a wave takes about (tiles per span + 2) tile
    times, the 2 standing for a block's start-up (its metadata, page ids and first tile arrive one
    after the other); every further span also costs a little in the merge.  The span with the
    lowest cost wins; measured on B200 at context 8192 this picks 1408 for batch 8 (384 blocks, one
    wave: 54 us against 58-66 us for spans of 384 to 1024) and 1664 for batch 64.  The kernels hold the
    same model (``pick_span_len``) and use it when they are given a span length of 0, with the step's
    own longest context; this function serves callers that fix the span themselves.
    """
    blocks_per_span = n_decode * n_kv_heads * ((n_q_heads // n_kv_heads + 15) // 16)
    slots = _slots(head_dim)
    tiles = max(1, (max_context + KV_TILE - 1) // KV_TILE)
    best, best_cost = 1, None
    for span_tiles in range(1, MAX_DECODE_SPAN // KV_TILE + 1):
        n_spans = (tiles + span_tiles - 1) // span_tiles
        waves = (blocks_per_span * n_spans + slots - 1) // slots
        cost = waves * (span_tiles + 2) + 0.15 * n_spans
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = span_tiles, cost
    return best * KV_TILE


def span_cap(n_decode, n_q_heads, n_kv_heads, max_context, head_dim=128) -> int:
    """The most spans the kernels may use for any context up to ``max_context`` when they choose the
    span length themselves (the grid's first dimension, and what the scratch is sized for).  The cost
    model never prefers a second wave of shorter spans to one wave, so one wave's worth of spans is
    enough unless the longest span (2048 positions) forces more."""
    slots, blocks_per_span = _slots(head_dim), n_decode * n_kv_heads * ((n_q_heads // n_kv_heads + 15) // 16)
    tiles = max(1, (max_context + KV_TILE - 1) // KV_TILE)
    longest = MAX_DECODE_SPAN // KV_TILE
    return min(tiles, max(-(-slots // blocks_per_span), -(-tiles // longest)) + 1)


def decode_scratch(ctx, n_decode, n_q_heads, n_spans, head_dim):
    """Partial sums and their (max, sum) pairs for the single-token kernel.

    One pair of buffers per runner, kept in ``ctx.extras`` (which the runner carries from step to
    step) and replaced by a larger pair when a step needs more; a recorded graph keeps the pair it
    was recorded with alive.
    """
    slots = n_decode * n_q_heads * n_spans
    scratch = ctx.extras.get("attn_decode_scratch")
    if scratch is None or scratch[0].numel() < slots * head_dim or scratch[1].numel() < slots * 2:
        grow = lambda old, need: max(need, 2 * old.numel() if old is not None else 0)
        old = scratch or (None, None)
        scratch = (torch.empty(grow(old[0], slots * head_dim), dtype=torch.float32, device=ctx.device),
                   torch.empty(grow(old[1], slots * 2), dtype=torch.float32, device=ctx.device))
        ctx.extras["attn_decode_scratch"] = scratch
    return scratch


def prefill(q, pages, out, tile_info, n_tiles, block_table, n_q_heads, n_kv_heads, head_dim, page_size, window,
            scale):
    """tile_info int32 [n_tiles * 4]: (first token, its position, rows <= 64, block-table row) per tile."""
    lib = library(head_dim)
    _check(lib, lib.qil_attn_prefill(
        _p(q), _p(pages), _p(out), _p(tile_info), c_int(n_tiles), _p(block_table), c_int(block_table.shape[1]),
        c_int(n_q_heads), c_int(n_kv_heads), c_int(page_size), c_int(pages.shape[0]), c_int(window),
        c_float(scale), _stream()), "attention (prompt portions)")


def decode(q, pages, out, decode_info, n_decode, part_o, part_ml, n_spans, span_len, block_table,
           n_q_heads, n_kv_heads, head_dim, page_size, window, scale):
    """decode_info int32 [n_decode * 4]: (token, its position, block-table row, 0) per single token."""
    lib = library(head_dim)
    _check(lib, lib.qil_attn_decode(
        _p(q), _p(pages), _p(out), _p(decode_info), c_int(n_decode), _p(part_o), _p(part_ml), c_int(n_spans),
        c_int(span_len), _p(block_table), c_int(block_table.shape[1]), c_int(n_q_heads), c_int(n_kv_heads),
        c_int(page_size), c_int(pages.shape[0]), c_int(window), c_float(scale), _stream()),
        "attention (single tokens)", kernels=2)


def projection_tail_usable(ctx, qkv, cache, n_q_heads, n_kv_heads, head_dim, rotary_dim, norm_weights) -> bool:
    """Can the single-token kernel take the projection's raw output (``attend_projection``)?  Every token of
    the step a single token of its request, bfloat16 throughout, at most 16 query heads per kv head."""
    return (ctx.n_decode == ctx.n_tokens and ctx.n_tiles == 0 and qkv.dtype == torch.bfloat16
            and cache.pages.dtype == torch.bfloat16 and supports(head_dim, n_q_heads, n_kv_heads)
            and n_q_heads // n_kv_heads <= 16 and rotary_dim % 4 == 0 and rotary_dim <= head_dim
            and all(w is None or w.dtype == torch.bfloat16 for w in norm_weights))


def attend_projection(ctx, qkv, cache, out, n_q_heads, n_kv_heads, own_kv_heads, head_dim, window, scale,
                      q_norm, k_norm, eps, rope_table, rotary_dim):
    """A step of single tokens, straight from the q/k/v projection: ``qkv`` bfloat16
    [N, (n_q_heads + 2 * own_kv_heads) * D].  The kernel norms and rotates the queries itself and writes
    each token's normed, rotated key and its value into the token's page before reading them, so the
    norm/rotation/store kernel is not launched.  ``own_kv_heads``: n_kv_heads, or 0 for a layer that
    reads another layer's cache."""
    if tuple(cache.pages.shape[1:]) != (2, n_kv_heads, cache.page_size, head_dim):
        raise KernelError(f"attention: cache layout {tuple(cache.pages.shape)}")
    if qkv.shape != (ctx.n_tokens, (n_q_heads + 2 * own_kv_heads) * head_dim) or not qkv.is_contiguous():
        raise KernelError(f"attention: projection output {tuple(qkv.shape)}")
    if rope_table is not None and (rope_table.dtype != torch.float32 or rope_table.shape[1] != rotary_dim
                                   or not rope_table.is_contiguous()):
        raise KernelError("attention: the rotary table must be float32 [positions, rotary_dim]")
    # the kernels pick the span from the step's own longest context (decode_info carries it); ctx.max_context
    # may be a recorded graph's upper bound and only caps the number of spans
    span_len, n_spans = 0, span_cap(ctx.n_decode, n_q_heads, n_kv_heads, ctx.max_context, head_dim)
    part_o, part_ml = decode_scratch(ctx, ctx.n_decode, n_q_heads, n_spans, head_dim)
    lib = library(head_dim)
    _check(lib, lib.qil_attn_decode_qkv(
        _p(qkv), _p(cache.pages), _p(out), _p(ctx.decode_info), c_int(ctx.n_decode), _p(part_o), _p(part_ml),
        c_int(n_spans), c_int(span_len), _p(cache.block_table), c_int(cache.block_table.shape[1]),
        c_int(n_q_heads), c_int(n_kv_heads), c_int(own_kv_heads), c_int(cache.page_size),
        c_int(cache.pages.shape[0]), c_int(window), c_float(scale), _p(q_norm), _p(k_norm), c_float(float(eps)),
        _p(rope_table), c_int(rotary_dim if rope_table is not None else 0),
        c_int(rope_table.shape[0] if rope_table is not None else 0), _stream()),
        "attention (single tokens from the projection)", kernels=2)


def attend(ctx, q, cache, out, n_q_heads, n_kv_heads, head_dim, window, scale):
    """q, out bfloat16 [N, Hq*D]; cache a KVCacheView whose pages already hold this step's keys and values."""
    if q.dtype != torch.bfloat16 or cache.pages.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention takes bfloat16 queries and pages")
    if tuple(cache.pages.shape[1:]) != (2, n_kv_heads, cache.page_size, head_dim):
        raise KernelError(f"attention: cache layout {tuple(cache.pages.shape)}")
    if ctx.n_big_tiles and attention_tc.supports(head_dim, cache.page_size, window):
        # whole 128-token tiles on tcgen05 with the accumulators in tensor memory, the leftovers below
        attention_tc.prefill(q, cache.pages, out, ctx.big_tile_info, ctx.n_big_tiles, cache.block_table,
                             n_q_heads, n_kv_heads, cache.page_size, scale)
        if ctx.n_rest_tiles:
            prefill(q, cache.pages, out, ctx.rest_tile_info, ctx.n_rest_tiles, cache.block_table, n_q_heads,
                    n_kv_heads, head_dim, cache.page_size, window, scale)
    elif ctx.n_tiles:
        prefill(q, cache.pages, out, ctx.tile_info, ctx.n_tiles, cache.block_table, n_q_heads, n_kv_heads,
                head_dim, cache.page_size, window, scale)
    if ctx.n_decode:
        span_len, n_spans = 0, span_cap(ctx.n_decode, n_q_heads, n_kv_heads, ctx.max_context, head_dim)
        part_o, part_ml = decode_scratch(ctx, ctx.n_decode, n_q_heads, n_spans, head_dim)
        decode(q, cache.pages, out, ctx.decode_info, ctx.n_decode, part_o, part_ml, n_spans, span_len,
               cache.block_table, n_q_heads, n_kv_heads, head_dim, cache.page_size, window, scale)
