"""Tensor-core attention for bfloat16, compiled per head size on first use.

``attend`` runs both forms over one step's batch: query tiles of prompt portions
go to the tiled kernel, single tokens to the span kernel plus its merge.  The
span kernel's partial sums live in scratch that is allocated once per step and
shared by all layers.
"""
from __future__ import annotations

import functools
from ctypes import c_float, c_int, c_void_p

import numpy as np
import torch

from . import attention_tc, build, tuning
from .ops import KernelError, _check, _p, _stream

_libs: dict = {}
KV_TILE = 64
MAX_DECODE_SPAN = 8192
QUERY_TILE = 64          # tokens per query tile of ``attn_prefill_kernel``
BIG_QUERY_TILE = attention_tc.TILE     # tokens per query tile of the tensor-memory kernel


PLAN_KEY = "paged_attention"     # the step planner whose arrays ``attend`` reads (``describe_segments`` makes them)


def describe_segments(first, starts, lens, rows) -> dict:
    """A step's segments as the attention kernels of this module and of ``attention_tc`` want them
    (numpy int64 arrays in, one entry per segment: first token in the flat batch, its absolute
    position, tokens, block-table row).

    ``tile_info``       query tiles of 64 tokens of every segment longer than one token; four ints a
                        tile: (first token in the flat batch, its absolute position, tokens in the tile,
                        block-table row)
    ``big_tile_info``   the same segments' whole tiles of 128 tokens (for the tensor-memory kernel) ...
    ``rest_tile_info``  ... and 64-token tiles of what those leave over (short segments, tails)
    ``decode_info``     segments of exactly one token: (token, its position, block-table row, the longest
                        context among these segments)

    Tiles are sorted with the longest contexts first: they take longest, the short ones fill the gaps.
    """
    def tiles(indices, tile, begin_of=lambda length: 0, end_of=lambda length: length):
        found = [(first[i] + off, starts[i] + off, min(tile, end_of(int(lens[i])) - off), rows[i])
                 for i in indices for off in range(begin_of(int(lens[i])), end_of(int(lens[i])), tile)]
        found.sort(key=lambda t: -(t[1] + t[2]))
        return np.array(found, dtype=np.int64).reshape(-1)

    multi = np.nonzero(lens > 1)[0]
    whole = lambda length: length // BIG_QUERY_TILE * BIG_QUERY_TILE
    single = np.nonzero(lens == 1)[0]
    if len(single):
        decode_info = np.stack([first[single], starts[single], rows[single],
                                np.full_like(single, int(starts[single].max()) + 1)], axis=1).reshape(-1)
    else:
        decode_info = np.zeros(0, dtype=np.int64)
    return dict(tile_info=tiles(multi, QUERY_TILE), big_tile_info=tiles(multi, BIG_QUERY_TILE, end_of=whole),
                rest_tile_info=tiles(multi, QUERY_TILE, begin_of=whole), decode_info=decode_info)


def refresh_single_tokens(arrays, starts) -> None:
    """``describe_segments`` of a step of single tokens whose rows are those of the step before:
    only the positions change (``arrays``: numpy views of the arrays made then, edited in place)."""
    info = arrays["decode_info"]
    n = len(starts)
    info[1:4 * n:4] = starts
    info[3:4 * n:4] = int(starts.max()) + 1


def step_plan(ctx):
    """The planner's arrays for the step in flight: (device arrays, their lengths)."""
    view = ctx.plans[PLAN_KEY]
    return view.array, view.count


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


# The span model, in "tile times" (what a block takes to stream a 64-key tile).  Blocks run in waves of
# (SMs x blocks per SM); a wave takes the tiles of a span plus SPAN_STARTUP for a block's start-up (its
# description, page ids and first tile arrive one after the other); every span costs the merge SPAN_MERGE.
# So the context is cut into as many spans as fill the GPU once, fewer when the requests are few.
# Measured inside the recorded decode step (Qwen3-8B heads, context 8192, B200): batch 8 takes 4.84 ms with
# 5 or 6 spans (320 or 384 of 444 slots), 4.97 with 4, 5.1 with 7 to 9 (a few blocks spill into a second
# wave), 4.92 with 11 to 13; batch 1 is flat from 16 to 43 spans, batch 4 best at 11, batch 16 at 3 or 6.
# Timed alone, without the projection before it and the chained launches around it, the same pair of
# kernels prefers fewer, longer spans (256 blocks: two per SM); that did not carry over to the step.
SPAN_STARTUP, SPAN_MERGE = tuning.SPAN_STARTUP_TILES, tuning.SPAN_MERGE_TILES


def _span_cost(tiles, n_spans, blocks_per_span, slots) -> float:
    """Tile times of the kernel pair for a longest context of ``tiles`` tiles cut into ``n_spans`` spans."""
    per_span = -(-tiles // n_spans)
    n_spans = -(-tiles // per_span)                     # spans that hold anything
    waves = -(-blocks_per_span * n_spans // slots)
    return waves * (per_span + SPAN_STARTUP) + SPAN_MERGE * n_spans


@functools.lru_cache(maxsize=4096)
def _plan_tiles(blocks_per_span, slots, lo, hi) -> int:
    """The number of spans with the lowest cost per tile at both ends of [lo, hi] tiles of longest context."""
    least = -(-hi // (MAX_DECODE_SPAN // KV_TILE))      # the longest span is a limit of the kernels
    best, best_cost = None, None
    for n_spans in range(least, max(least, min(hi, 256)) + 1):
        cost = _span_cost(hi, n_spans, blocks_per_span, slots) / hi
        if lo != hi:
            cost += _span_cost(lo, min(n_spans, lo), blocks_per_span, slots) / lo
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = n_spans, cost
    return best


def plan_spans(n_decode, n_q_heads, n_kv_heads, max_context, head_dim=128, min_context=None, slots=None):
    """(n_spans, longest span) for steps whose longest context lies in [min_context, max_context]: the kernels
    cut each step's own longest context into ``n_spans`` equal spans (a recorded graph is replayed while
    contexts grow), so the count is chosen for both ends of the range; the longest span sizes shared memory.
    Eager steps ask once per layer and step: the answer is remembered per (blocks, tiles).  ``slots``: how many
    blocks run at a time, when it is not this module's span kernel that runs them."""
    blocks_per_span = n_decode * n_kv_heads * ((n_q_heads // n_kv_heads + 15) // 16)
    hi = max(1, (max_context + KV_TILE - 1) // KV_TILE)
    lo = max(1, min(hi, ((min_context or max_context) + KV_TILE - 1) // KV_TILE))
    n_spans = _plan_tiles(blocks_per_span, slots or _slots(head_dim), lo, hi)
    return n_spans, -(-hi // n_spans) * KV_TILE


def choose_span(n_decode, n_q_heads, n_kv_heads, max_context, head_dim=128) -> int:
    """Positions per block of the single-token kernel for a step whose longest context is ``max_context``."""
    return plan_spans(n_decode, n_q_heads, n_kv_heads, max_context, head_dim)[1]


def merge_in_kernel(n_decode, n_q_heads, n_kv_heads, head_dim) -> bool:
    """Should the span kernel's blocks merge their spans themselves (the last block of a token's spans, found
    by a ticket counter) instead of leaving it to a second kernel?  A ticket costs every block a fence and an
    atomic at its end; a merge kernel costs a launch between the attention and the output projection.  With
    few tokens the launch is what shows, with many (a span's worth of blocks fills the GPU) the tickets are."""
    import os
    blocks_per_span = n_decode * n_kv_heads * ((n_q_heads // n_kv_heads + 15) // 16)
    return blocks_per_span <= int(os.environ.get("QIL_TICKET_MAX_BLOCKS", _slots(head_dim)))


def decode_scratch(ctx, n_decode, n_q_heads, n_spans, head_dim):
    """Partial sums, their (max, sum) pairs and the ticket counters for the single-token kernel (the blocks
    of a token's spans count themselves in, the last one merges; the counters are zero between launches).

    One pair of buffers per runner, kept in ``ctx.extras`` (which the runner carries from step to
    step) and replaced by a larger pair when a step needs more; a recorded graph keeps the pair it
    was recorded with alive.
    """
    slots = n_decode * n_q_heads * n_spans
    scratch = ctx.extras.get("attn_decode_scratch")
    # one counter per (token, kv head, chunk of 16 query heads) at most: a counter per query head is always enough
    if scratch is None or scratch[0].numel() < slots * head_dim or scratch[1].numel() < slots * 2 \
            or len(scratch) < 3 or scratch[2].numel() < n_decode * n_q_heads:
        grow = lambda old, need: max(need, 2 * old.numel() if old is not None else 0)
        old = (tuple(scratch) + (None, None, None))[:3] if scratch else (None, None, None)
        scratch = (torch.empty(grow(old[0], slots * head_dim), dtype=torch.float32, device=ctx.device),
                   torch.empty(grow(old[1], slots * 2), dtype=torch.float32, device=ctx.device),
                   torch.zeros(grow(old[2], n_decode * n_q_heads), dtype=torch.int32, device=ctx.device))
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
           n_q_heads, n_kv_heads, head_dim, page_size, window, scale, tickets=None):
    """decode_info int32 [n_decode * 4]: (token, its position, block-table row, the step's longest context)
    per single token.  A negative ``span_len``: the kernels cut the step's longest context into ``n_spans``
    equal spans of at most ``-span_len`` positions (see ``plan_spans``).  ``tickets``: int32 zeros, one per
    (token, query head) or more (``decode_scratch``): the last block of a token's spans merges them; None: a
    second kernel does."""
    lib = library(head_dim)
    _check(lib, lib.qil_attn_decode(
        _p(q), _p(pages), _p(out), _p(decode_info), c_int(n_decode), _p(part_o), _p(part_ml), _p(tickets), c_int(n_spans),
        c_int(span_len), _p(block_table), c_int(block_table.shape[1]), c_int(n_q_heads), c_int(n_kv_heads),
        c_int(page_size), c_int(pages.shape[0]), c_int(window), c_float(scale), _stream()),
        "attention (single tokens)", kernels=1 if tickets is not None else 2)


def projection_tail_usable(ctx, qkv, cache, n_q_heads, n_kv_heads, head_dim, rotary_dim, norm_weights) -> bool:
    """Can the single-token kernel take the projection's raw output (``attend_projection``)?  Every token of
    the step a single token of its request, bfloat16 throughout, at most 16 query heads per kv head."""
    return (step_plan(ctx)[1]["decode_info"] == 4 * ctx.n_tokens and qkv.dtype == torch.bfloat16
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
    # the kernels cut the step's own longest context (decode_info carries it) into n_spans spans; ctx.max_context
    # may be a recorded graph's upper bound, ctx.min_context its lower one
    arrays, counts = step_plan(ctx)
    n_decode = counts["decode_info"] // 4
    n_spans, longest_span = plan_spans(n_decode, n_q_heads, n_kv_heads, ctx.max_context, head_dim,
                                       getattr(ctx, "min_context", 0) or None)
    part_o, part_ml, tickets = decode_scratch(ctx, n_decode, n_q_heads, n_spans, head_dim)
    if not merge_in_kernel(n_decode, n_q_heads, n_kv_heads, head_dim):
        tickets = None
    lib = library(head_dim)
    _check(lib, lib.qil_attn_decode_qkv(
        _p(qkv), _p(cache.pages), _p(out), _p(arrays["decode_info"]), c_int(n_decode), _p(part_o), _p(part_ml),
        _p(tickets), c_int(n_spans), c_int(-longest_span), _p(cache.block_table), c_int(cache.block_table.shape[1]),
        c_int(n_q_heads), c_int(n_kv_heads), c_int(own_kv_heads), c_int(cache.page_size),
        c_int(cache.pages.shape[0]), c_int(window), c_float(scale), _p(q_norm), _p(k_norm), c_float(float(eps)),
        _p(rope_table), c_int(rotary_dim if rope_table is not None else 0),
        c_int(rope_table.shape[0] if rope_table is not None else 0), _stream()),
        "attention (single tokens from the projection)", kernels=1 if tickets is not None else 2)


def attend(ctx, q, cache, out, n_q_heads, n_kv_heads, head_dim, window, scale):
    """q, out bfloat16 [N, Hq*D]; cache a KVCacheView whose pages already hold this step's keys and values."""
    if q.dtype != torch.bfloat16 or cache.pages.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention takes bfloat16 queries and pages")
    if tuple(cache.pages.shape[1:]) != (2, n_kv_heads, cache.page_size, head_dim):
        raise KernelError(f"attention: cache layout {tuple(cache.pages.shape)}")
    arrays, counts = step_plan(ctx)
    n_tiles, n_big, n_rest, n_decode = (counts[name] // 4 for name in
                                        ("tile_info", "big_tile_info", "rest_tile_info", "decode_info"))
    if n_big and attention_tc.supports(head_dim, cache.page_size, window):
        # whole 128-token tiles on tcgen05 with the accumulators in tensor memory, the leftovers below
        attention_tc.prefill(q, cache.pages, out, arrays["big_tile_info"], n_big, cache.block_table,
                             n_q_heads, n_kv_heads, cache.page_size, scale)
        if n_rest:
            prefill(q, cache.pages, out, arrays["rest_tile_info"], n_rest, cache.block_table, n_q_heads,
                    n_kv_heads, head_dim, cache.page_size, window, scale)
    elif n_tiles:
        prefill(q, cache.pages, out, arrays["tile_info"], n_tiles, cache.block_table, n_q_heads, n_kv_heads,
                head_dim, cache.page_size, window, scale)
    if n_decode:
        n_spans, longest_span = plan_spans(n_decode, n_q_heads, n_kv_heads, ctx.max_context, head_dim,
                                           getattr(ctx, "min_context", 0) or None)
        part_o, part_ml, tickets = decode_scratch(ctx, n_decode, n_q_heads, n_spans, head_dim)
        if not merge_in_kernel(n_decode, n_q_heads, n_kv_heads, head_dim):
            tickets = None
        decode(q, cache.pages, out, arrays["decode_info"], n_decode, part_o, part_ml, n_spans, -longest_span,
               cache.block_table, n_q_heads, n_kv_heads, head_dim, cache.page_size, window, scale, tickets)
