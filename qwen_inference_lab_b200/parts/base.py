"""What every part of a model is made of: parameters, cache needs, the step context.

A model is a tree of parts.  A part owns its sizes and constants (given as
arguments, never read from a global configuration), its parameters, and a
``forward`` over the flat batch of tokens that one step brings.  No part knows
which model it is in: the checkpoint names of its parameters are handed to it by
the architecture's builder.

Interfaces
----------
``Part``        ``named_params()`` (checkpoint name -> ``Param``), ``children()``,
                ``finalize(device, dtype)`` after the weights are in.
``Norm``        ``forward(ctx, x, rows=None) -> y`` over the last dimension.
``PositionEncoding``  ``table`` (float32 ``[positions, rotary_dim]``: cosines then
                sines) and ``rotary_dim``; mixers hand the table to their kernels.
``Mixer``       ``cache_spec()`` (what it keeps per request: paged keys/values, a
                fixed-size state, or nothing) and ``forward(ctx, x, cache, residual=None) -> y``.
``FeedForward`` ``forward(ctx, x, residual=None) -> y``.
                A mixer or feed-forward with ``takes_norm = True`` is handed the block's
                un-normed input and the norm (``norm=``) and applies it itself, so that it can
                fuse the norm into its first product; the others get normed input.
``Block``       ``forward(ctx, x, cache) -> x`` (arrangement of the above).
``StepPlanner`` what a part's kernels need to know about a step beyond its segments (query
                tiles, work lists): computed on the host from ``Segments``, packed and uploaded by
                the step function with everything else, handed back in ``ctx.plans[key]``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


class Param:
    """One parameter tensor: shape, how random weights draw it, and the loaded data.

    ``init`` is ``"normal"`` (N(0, std)), ``"norm"`` (1 + N(0, std)) or ``"zeros"``.
    Several checkpoint names may point to one Param (tied embeddings).
    ``keep_32bit``: a tensor that the checkpoint stores in 32 bits stays so in a bfloat16 run (for
    parameters whose part computes in float32, such as router weights or decay rates); all others
    are cast to the run's dtype when they are loaded, as the reference does (qil/model.py:197).
    """

    __slots__ = ("shape", "init", "std", "data", "integer", "keep_32bit")

    def __init__(self, shape, init="normal", std=0.02, integer=False, keep_32bit=False):
        self.shape = tuple(int(n) for n in shape)
        self.init = init
        self.std = std
        self.integer = integer
        self.keep_32bit = keep_32bit
        self.data: torch.Tensor | None = None

    def __repr__(self):
        return f"Param{self.shape}"


@dataclass(frozen=True)
class KVCacheSpec:
    """Paged keys and values: ``kv_heads * head_dim`` of each per token.

    ``window`` > 0 means that only the last ``window`` positions are ever read, so
    pages that the window has passed are given back while the request lives.
    """
    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """A fixed-size state per request (``shape`` elements of ``dtype``), zeroed at admission."""
    shape: tuple
    dtype: torch.dtype = torch.float32


class Part:
    """Base of all parts."""

    #: True when ``forward`` only launches work on the current stream with no host
    #: synchronisation and no data-dependent host control flow, so that a step made
    #: of such parts may be recorded into a CUDA graph.
    graph_safe = False

    def named_params(self) -> dict:
        """Checkpoint name -> Param for this part alone (children excluded)."""
        return {}

    def children(self) -> list:
        return []

    def all_named_params(self) -> dict:
        result = dict(self.named_params())
        for child in self.children():
            for name, param in child.all_named_params().items():
                if name in result and result[name] is not param:
                    raise ValueError(f"two different parameters claim the name {name}")
                result[name] = param
        return result

    def finalize(self, device, dtype) -> None:
        """Called once after all parameters hold data; fuse or derive tensors here."""
        for child in self.children():
            child.finalize(device, dtype)

    def is_graph_safe(self) -> bool:
        return self.graph_safe and all(child.is_graph_safe() for child in self.children())

    def step_planners(self) -> dict:
        """key -> StepPlanner for this part and its children.  Parts that give the same key share one
        plan per step (all attention layers of a model read the same query tiles)."""
        result = {}
        for child in self.children():
            result.update(child.step_planners())
        return result


class Norm(Part):
    def forward(self, ctx, x, rows=None):
        raise NotImplementedError

    def as_rms(self):
        """(weight tensor, eps) if this norm is a plain root-mean-square norm that a product kernel
        may apply itself, else None."""
        return None


class PositionEncoding(Part):
    rotary_dim = 0
    table: torch.Tensor | None = None


class Mixer(Part):
    def cache_spec(self):
        return None

    def forward(self, ctx, x, cache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x, residual=None):
        raise NotImplementedError


@dataclass
class Segments:
    """The batch of one step as the host sees it (numpy int64 arrays, one entry per segment).

    A segment is one request's run of consecutive tokens in the flat batch.  This is all the
    step function knows about a batch; whatever else a kernel wants (tiles of its own size, lists
    of single tokens) a ``StepPlanner`` derives from it.
    """
    rows: object        # [S] request row (block-table row, state slot)
    first: object       # [S] index of the segment's first token in the flat batch
    lens: object        # [S] tokens in the segment
    starts: object      # [S] absolute position of the segment's first token
    n_tokens: int

    @property
    def n_segments(self) -> int:
        return len(self.lens)


class StepPlanner:
    """Host-side planning of a step for one family of kernels.

    ``plan`` returns named integer arrays; the step function packs them (as int32) into the step's
    one upload and gives the part device views of them: ``ctx.plans[key].array[name]`` with
    ``ctx.plans[key].count[name]`` entries.  For a step in which every segment is a single token
    the length of every array may depend on the number of segments only, not on positions or
    rows: such steps are recorded into CUDA graphs that are replayed with other positions.

    ``refresh_single_tokens`` is optional: when consecutive steps bring one token each for the same
    requests in the same rows, only positions change, and a planner that can overwrite just those
    in its arrays of the previous step (numpy views, edited in place) returns True; returning
    False makes the step function call ``plan`` again.
    """
    key = ""

    def plan(self, segments: Segments) -> dict:
        raise NotImplementedError

    def refresh_single_tokens(self, arrays: dict, segments: Segments) -> bool:
        return False


@dataclass
class PlanView:
    """A planner's arrays as the parts see them: int32 device views and their lengths."""
    array: dict = field(default_factory=dict)
    count: dict = field(default_factory=dict)


@dataclass
class StepContext:
    """Everything a part may know about the step in flight.

    The batch is flat: ``n_tokens`` tokens made of ``n_segments`` segments, one per
    request, each a run of consecutive positions.  Device arrays are int32.
    Host copies (``h_*``, numpy) describe the same batch for parts that plan on
    the host; graph-safe parts read the device arrays only.
    """
    n_tokens: int
    n_segments: int
    dtype: torch.dtype
    device: torch.device
    token_ids: torch.Tensor          # [N]
    positions: torch.Tensor          # [N] absolute position of each token
    token_row: torch.Tensor          # [N] request slot (row of block tables / state slots)
    seg_row: torch.Tensor            # [S] request slot of each segment
    seg_start: torch.Tensor          # [S] first token of the segment in the flat batch
    seg_len: torch.Tensor            # [S]
    seg_pos0: torch.Tensor           # [S] position of the segment's first token
    max_context: int                 # largest start+len over the batch's segments (host upper bound)
    # a recorded graph is replayed with other contexts than the step it was recorded from: max_context is then
    # the largest longest-context of those steps and min_context the smallest (0: this step only)
    min_context: int = 0
    # key -> PlanView: what the model's step planners made of this step's segments
    plans: dict = field(default_factory=dict)
    h_seg_row: object = None
    h_seg_start: object = None
    h_seg_len: object = None
    h_seg_pos0: object = None
    # the runner's own dict, the same one every step: parts keep scratch buffers here under their own keys
    extras: dict = field(default_factory=dict)

    def empty(self, shape, dtype=None):
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)
