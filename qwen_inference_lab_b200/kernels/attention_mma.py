"""Tensor-core attention kernels for bfloat16 (compiled per head size on first use)."""
from __future__ import annotations


def supports(head_dim, n_q_heads, n_kv_heads) -> bool:
    return False


def attend(ctx, q, cache, out, n_q_heads, n_kv_heads, head_dim, window, scale):
    raise NotImplementedError
