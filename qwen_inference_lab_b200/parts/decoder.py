"""A decoder-only language model as data: parts, and the order in which layers run.

``layers`` is a list of blocks; ``order`` is a list of :class:`LayerCall`, each
naming a layer by index.  A layer may be named twice (its weights are shared, each
call keeps a cache of its own), and a call may read the cache that an earlier
call wrote instead of owning one.  The model knows nothing of requests or pages:
it is handed one cache view per call and the step's context.

Embedding, final norm and head follow the reference's ``Qwen3`` (qil/model.py:89-98,
126-134): rows are looked up in the activation dtype, the final norm and the head
run only for the positions whose logits were asked for, logits are float32.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..kernels import ops
from .base import Param, Part
from .linear import Linear


@dataclass(frozen=True)
class LayerCall:
    """One entry of the order: run ``layer``; ``reads_cache_of`` is the index (into the
    order) of the earlier call whose cache this call reads, or None to own one."""
    layer: int
    reads_cache_of: int | None = None


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab_size, hidden_size, *, name):
        self.vocab_size, self.hidden_size, self.name = int(vocab_size), int(hidden_size), name
        self.weight = Param((vocab_size, hidden_size))

    def named_params(self):
        return {self.name + ".weight": self.weight}

    def forward(self, ctx, token_ids):
        out = ctx.empty((token_ids.shape[0], self.hidden_size))
        return ops.embed_gather(self.weight.data, token_ids, out)


class DecoderModel(Part):
    graph_safe = True      # the model itself only walks its parts; they decide

    def __init__(self, *, config, embedding, layers, order, final_norm, head, max_positions):
        self.config = config
        self.embedding, self.layers, self.final_norm, self.head = embedding, list(layers), final_norm, head
        self.order = [call if isinstance(call, LayerCall) else LayerCall(*call) for call in order]
        self.max_positions = int(max_positions)
        self.vocab_size = embedding.vocab_size
        self.device = None
        self.dtype = None
        for index, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"order[{index}] names layer {call.layer} of {len(self.layers)}")
            owns = self.layers[call.layer].cache_spec() is not None
            if call.reads_cache_of is not None:
                source = call.reads_cache_of
                if not 0 <= source < index or self.order[source].reads_cache_of is not None \
                        or self.layers[self.order[source].layer].cache_spec() is None:
                    raise ValueError(f"order[{index}] must read the cache of an earlier call that owns one")
                if owns:
                    raise ValueError(f"order[{index}]: a layer that keeps its own cache cannot read another's")

    def children(self):
        return [self.embedding, *self.layers, self.final_norm, self.head]

    def cache_specs(self):
        """One entry per call of the order: the cache it owns, or None."""
        return [None if call.reads_cache_of is not None else self.layers[call.layer].cache_spec()
                for call in self.order]

    def finalize(self, device, dtype):
        self.device, self.dtype = torch.device(device), dtype
        super().finalize(device, dtype)

    def forward(self, ctx, cache_views, logit_rows, checkpoint=None, calls_per_checkpoint=12):
        """Run the batch through every call of the order; float32 logits [R, vocab] or None.

        ``cache_views[i]`` is the view for order[i] (its own cache, or the one it reads);
        ``logit_rows`` int32 [R] indexes the flat batch (None or empty: no logits).
        ``checkpoint`` is called between groups of layer calls: whoever records the step into
        CUDA graphs cuts there, so that the GPU starts on the first layers while the rest is
        still being submitted.
        """
        x = self.embedding.forward(ctx, ctx.token_ids)
        for index, call in enumerate(self.order):
            if checkpoint is not None and index and index % calls_per_checkpoint == 0:
                checkpoint()
            x = self.layers[call.layer].forward(ctx, x, cache_views[index])
        if logit_rows is None or logit_rows.shape[0] == 0:
            return None
        normed = self.final_norm.forward(ctx, x, rows=logit_rows)
        return self.head.forward(ctx, normed, out_float32=True)
