"""Causal grouped-query attention over paged keys and values.

Per token: q, k, v projections (one stacked product), RMSNorm of every q and k
head over head_dim, rotation of q and k by the token's absolute position, k and v
written to the request's pages, softmax(q k^T * scale) over the keys up to the
token's own position (inside the window, if one is set), times v, then the output
projection (qil/model.py:48-69 for a chunk, :73-84 for single tokens; both are
the same computation here, every token of the flat batch takes it).  Query head
``h`` reads kv head ``h // (n_q_heads // n_kv_heads)`` (qil/paged_attention.py:21).
"""
from __future__ import annotations

import torch

from ..kernels import attention_mma, gemm_tc, ops
from .base import KVCacheSpec, Mixer, Param, StepPlanner
from .linear import Linear, StackedLinear


class PagedAttentionPlanner(StepPlanner):
    """The host hook of the attention mixers: a step's segments cut into the query tiles and the list
    of single tokens that the attention kernels take (``attention_mma.describe_segments``).  All
    attention layers of a model share the one plan."""
    key = attention_mma.PLAN_KEY

    def plan(self, segments):
        return attention_mma.describe_segments(segments.first, segments.starts, segments.lens, segments.rows)

    def refresh_single_tokens(self, arrays, segments):
        attention_mma.refresh_single_tokens(arrays, segments.starts)
        return True


_PLANNER = PagedAttentionPlanner()


class GroupedQueryAttention(Mixer):
    """Sizes and constants are arguments; ``names`` gives the checkpoint names.

    names: dict with keys q, k, v, o (projection names, without ``.weight``) and,
    when ``qk_norm_eps`` is not None, q_norm and k_norm.
    ``reads_shared_cache=True`` builds a layer without k and v projections that
    attends over pages another layer wrote (the model's order says which).
    """
    graph_safe = True

    def __init__(self, hidden_size, n_q_heads, n_kv_heads, head_dim, *, names, bias=False,
                 qk_norm_eps=None, position=None, window=0, scale=None, reads_shared_cache=False):
        if n_q_heads % n_kv_heads:
            raise ValueError(f"{n_q_heads} query heads do not divide into {n_kv_heads} kv heads")
        self.hidden_size, self.head_dim = int(hidden_size), int(head_dim)
        self.n_q_heads, self.n_kv_heads = int(n_q_heads), int(n_kv_heads)
        self.window = int(window)
        self.scale = float(scale) if scale is not None else float(head_dim) ** -0.5
        self.qk_norm_eps = qk_norm_eps
        self.position = position
        self.reads_shared_cache = bool(reads_shared_cache)
        pieces = [(names["q"], n_q_heads * head_dim)]
        if not self.reads_shared_cache:
            pieces += [(names["k"], n_kv_heads * head_dim), (names["v"], n_kv_heads * head_dim)]
        self.qkv = StackedLinear(hidden_size, pieces, bias=bias)
        self.out = Linear(n_q_heads * head_dim, hidden_size, name=names["o"], bias=bias)
        self.q_norm = self.k_norm = None
        self._norm_names = None
        if qk_norm_eps is not None:
            self.q_norm = Param((head_dim,), init="norm", std=0.05)
            self.k_norm = Param((head_dim,), init="norm", std=0.05)
            self._norm_names = (names["q_norm"] + ".weight", names["k_norm"] + ".weight")

    def named_params(self):
        if self._norm_names is None:
            return {}
        return {self._norm_names[0]: self.q_norm, self._norm_names[1]: self.k_norm}

    def children(self):
        parts = [self.qkv, self.out]
        if self.position is not None:
            parts.append(self.position)
        return parts

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        if self.q_norm is not None and self.q_norm.data.dtype != self.k_norm.data.dtype:
            self.q_norm.data, self.k_norm.data = self.q_norm.data.float(), self.k_norm.data.float()

    def step_planners(self):
        return {**super().step_planners(), _PLANNER.key: _PLANNER}

    def cache_spec(self):
        if self.reads_shared_cache:
            return None
        return KVCacheSpec(self.n_kv_heads, self.head_dim, self.window)

    takes_norm = True

    def forward(self, ctx, x, cache, residual=None, norm=None):
        """x [N, hidden] -> [N, hidden] (+ residual).  ``cache`` is a KVCacheView.  With ``norm`` x is
        the block's un-normed input and the first projection applies the norm."""
        n = x.shape[0]
        n_kv = 0 if self.reads_shared_cache else self.n_kv_heads
        table = self.position.table if self.position is not None else None
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        q_norm = self.q_norm.data if self.q_norm is not None else None
        k_norm = self.k_norm.data if self.k_norm is not None else None
        if gemm_tc.qkv_tail_usable(x, self.qkv._weight(), self.head_dim, rotary_dim, (q_norm, k_norm), cache.pages):
            # long prompt portions: one tcgen05 kernel projects, norms, rotates and writes the pages
            if norm is not None:
                x = norm.forward(ctx, x)
            q = ctx.empty((n, self.n_q_heads * self.head_dim))
            gemm_tc.gemm_tc_qkv(x, self.qkv._weight(), self.qkv._bias(), q, cache.pages, table, q_norm, k_norm,
                                self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, ctx.positions,
                                ctx.token_row, cache.block_table, self.n_q_heads, n_kv, cache.page_size)
            attended = ctx.empty((n, self.n_q_heads * self.head_dim))
            self._attend(ctx, q, cache, attended)
            return self.out.forward(ctx, attended, residual=residual)
        qkv = self.qkv.forward(ctx, x, norm=norm)
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        if attention_mma.projection_tail_usable(ctx, qkv, cache, self.n_q_heads, self.n_kv_heads, self.head_dim,
                                                rotary_dim, (q_norm, k_norm)):
            # a step of single tokens: the attention kernel norms, rotates and stores what it needs itself
            attended = ctx.empty((n, self.n_q_heads * self.head_dim))
            attention_mma.attend_projection(ctx, qkv, cache, attended, self.n_q_heads, self.n_kv_heads, n_kv,
                                            self.head_dim, self.window, self.scale, q_norm, k_norm, eps, table,
                                            rotary_dim)
            return self.out.forward(ctx, attended, residual=residual)
        q = ctx.empty((n, self.n_q_heads * self.head_dim))
        ops.qk_norm_rope_store(qkv, q, cache.pages, q_norm, k_norm, eps, table, rotary_dim, ctx.positions,
                               ctx.token_row, cache.block_table, self.n_q_heads, n_kv, self.head_dim, cache.page_size)
        attended = ctx.empty((n, self.n_q_heads * self.head_dim))
        self._attend(ctx, q, cache, attended)
        return self.out.forward(ctx, attended, residual=residual)

    def _attend(self, ctx, q, cache, out):
        if q.dtype == torch.bfloat16 and attention_mma.supports(self.head_dim, self.n_q_heads, self.n_kv_heads):
            attention_mma.attend(ctx, q, cache, out, self.n_q_heads, self.n_kv_heads, self.head_dim,
                                 self.window, self.scale)
            return
        ops.attention_generic(q, cache.pages, out, ctx.positions, ctx.token_row, cache.block_table,
                              self.n_q_heads, self.n_kv_heads, self.head_dim, cache.page_size,
                              self.window, self.scale)
