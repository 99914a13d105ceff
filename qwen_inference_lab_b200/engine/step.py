"""The step function: one flat batch of (request, its next tokens) through the model.

A step takes any mix of prompt portions and single decoded tokens, cut anywhere,
runs exactly those tokens as one batch against the cache that earlier steps
left, and returns float32 logits at the places that were asked for.  The
reference runs a prefill chunk of one request (qil/model.py:110-134) or one token
of several requests (qil/model.py:136-157) per forward and several forwards per
step (qil/engine.py:63-86); here every step is one pass over the layers.

The batch is described to the kernels by int32 arrays in one device buffer,
uploaded with a single copy per step (see :class:`StepContext` for the fields).
Steps made only of single tokens are recorded into CUDA graphs, one per batch
size and context bucket, and replayed after the metadata upload.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..kernels import ops
from ..parts.base import StepContext
from ..utils.staging import PinnedRing

QUERY_TILE = 64          # tokens per query tile of the prompt-portion attention kernel
BIG_QUERY_TILE = 128     # tokens per query tile of the tensor-memory attention kernel


class StepError(ValueError):
    """A batch that cannot run: unknown request, bad token, position beyond the context..."""


PENDING = -1      # in ``StepEntry.tokens``: a token that is still on the device (see ``StepEntry.feed``)


@dataclass
class StepEntry:
    request_id: object
    tokens: list
    want: list = field(default_factory=list)   # indices into ``tokens`` whose logits are returned
    # When the last of ``tokens`` is PENDING: its index in the device buffer given to ``run`` as
    # ``token_source`` (the tokens that the step before sampled and the host has not read yet).
    feed: int | None = None


def _align4(n):
    return (n + 3) & ~3


class StepRunner:
    def __init__(self, model, cache, *, max_step_tokens=4096, use_graphs=True, graph_max_batch=256):
        self.model, self.cache = model, cache
        self.device = model.device
        self.views = cache.views(model.order)
        self.use_graphs = bool(use_graphs) and self.device.type == "cuda" and model.is_graph_safe()
        self.graph_max_batch = graph_max_batch
        self._capacity = 0
        self._meta_dev = None
        self._ring = PinnedRing() if self.device.type == "cuda" else None
        self._graphs: dict = {}
        self._graph_pool = None
        self._extras: dict = {}      # what parts keep from step to step (scratch buffers), by their own keys
        self._single_token_template = None
        self._reserve(8 * max_step_tokens + 16 * cache.max_requests + 64)
        self.steps_run = 0
        self.kernel_launches = 0          # this engine's own kernels (library products are not counted)
        self.launches_per_graph: dict = {}
        self.last_upload_bytes = 0

    def _reserve(self, ints):
        if ints <= self._capacity:
            return
        self._capacity = int(ints)
        self._meta_dev = torch.zeros(self._capacity, dtype=torch.int32, device=self.device)
        self._graphs.clear()     # recorded graphs point into the old buffer
        self._graph_pool = None  # their memory pool goes with the last of them: the next recording starts a new one

    # ------------------------------------------------------------------ the batch
    def _validate(self, entries):
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        vocab = self.model.vocab_size
        for entry in entries:
            if entry.request_id in seen:
                raise StepError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            if entry.request_id not in self.cache.rows:
                raise StepError(f"request {entry.request_id!r} has not been admitted to the cache")
            tokens = entry.tokens
            if len(tokens) == 0:
                raise StepError(f"request {entry.request_id!r} brings no tokens")
            known = tokens if entry.feed is None else tokens[:-1]
            if any(type(t) is not int or not 0 <= t < vocab for t in known):
                raise StepError(f"request {entry.request_id!r}: token ids must be integers in [0, {vocab})")
            if entry.feed is not None and (tokens[-1] != PENDING or type(entry.feed) is not int or entry.feed < 0):
                raise StepError(f"request {entry.request_id!r}: a fed token must be the last one and marked PENDING")
            start = self.cache.written(entry.request_id)
            if start + len(tokens) > self.model.max_positions:
                raise StepError(f"request {entry.request_id!r} exceeds the model's {self.model.max_positions} positions")
            if any(type(w) is not int or not 0 <= w < len(tokens) for w in entry.want):
                raise StepError(f"request {entry.request_id!r}: wanted places must index its tokens of this step")

    def _describe_single_tokens(self, entries):
        """The description of a step in which every request brings one token.  Consecutive decode steps
        of the same requests differ only in the tokens and the positions: the packed vector of the last
        such step is kept and those entries are overwritten."""
        key = tuple((e.request_id, tuple(e.want), e.feed) for e in entries)
        starts = np.fromiter((self.cache.written(e.request_id) for e in entries), dtype=np.int64, count=len(entries))
        kept = self._single_token_template
        if kept is None or kept[0] != key:
            packed, offsets, host, n, s, _ = self._describe_general(entries)
            self._single_token_template = kept = (key, packed, offsets, host)
        _, packed, offsets, host = kept
        n = len(entries)
        begin = offsets["token_ids"][0]
        packed[begin:begin + n] = [e.tokens[0] for e in entries]
        for name in ("positions", "seg_pos0"):
            begin = offsets[name][0]
            packed[begin:begin + n] = starts
        longest = int(starts.max()) + 1
        begin = offsets["decode_info"][0]
        packed[begin + 1:begin + 4 * n:4] = starts
        packed[begin + 3:begin + 4 * n:4] = longest
        host = dict(host, seg_pos0=starts)
        return packed, offsets, host, n, n, longest

    def _describe(self, entries):
        """Host arrays of the batch, packed into one int32 vector with section offsets."""
        if all(len(e.tokens) == 1 for e in entries):
            return self._describe_single_tokens(entries)
        return self._describe_general(entries)

    def _describe_general(self, entries):
        lens = np.array([len(e.tokens) for e in entries], dtype=np.int64)
        starts = np.array([self.cache.written(e.request_id) for e in entries], dtype=np.int64)
        rows = np.array([self.cache.row(e.request_id) for e in entries], dtype=np.int64)
        n, s = int(lens.sum()), len(entries)
        seg_start = np.zeros(s, dtype=np.int64)
        np.cumsum(lens[:-1], out=seg_start[1:])
        token_ids = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=n)
        seg_of_token = np.repeat(np.arange(s), lens)
        positions = np.arange(n) - seg_start[seg_of_token] + starts[seg_of_token]
        token_row = rows[seg_of_token]
        logit_rows = np.array([seg_start[i] + w for i, e in enumerate(entries) for w in e.want], dtype=np.int64)
        # query tiles of segments longer than one token: (first token, its position, rows, block-table row)
        tiles = [(seg_start[i] + off, starts[i] + off, min(QUERY_TILE, int(lens[i]) - off), rows[i])
                 for i in np.nonzero(lens > 1)[0] for off in range(0, int(lens[i]), QUERY_TILE)]
        # the longest tiles of the longest contexts first: they take longest, the short ones fill the gaps
        tiles.sort(key=lambda t: -(t[1] + t[2]))
        tile_info = np.array(tiles, dtype=np.int64).reshape(-1)
        # the same tokens cut for kernels that take whole tiles of 128 tokens: those tiles, and 64-token
        # tiles for what they leave over (short segments and the tails of long ones)
        big, rest = [], []
        for i in np.nonzero(lens > 1)[0]:
            whole = int(lens[i]) // BIG_QUERY_TILE * BIG_QUERY_TILE
            big += [(seg_start[i] + off, starts[i] + off, BIG_QUERY_TILE, rows[i]) for off in range(0, whole, BIG_QUERY_TILE)]
            rest += [(seg_start[i] + off, starts[i] + off, min(QUERY_TILE, int(lens[i]) - off), rows[i])
                     for off in range(whole, int(lens[i]), QUERY_TILE)]
        big.sort(key=lambda t: -(t[1] + t[2]))
        rest.sort(key=lambda t: -(t[1] + t[2]))
        big_tile_info = np.array(big, dtype=np.int64).reshape(-1)
        rest_tile_info = np.array(rest, dtype=np.int64).reshape(-1)
        # single-token segments: (token, its position, block-table row, the longest context among them)
        single = np.nonzero(lens == 1)[0]
        decode_info = np.stack([seg_start[single], starts[single], rows[single],
                                np.full_like(single, int(starts[single].max()) + 1)],
                               axis=1).reshape(-1) if len(single) else np.zeros(0, dtype=np.int64)
        # places of tokens that are still on the device: (index in the flat batch, index in the source buffer)
        feed = np.array([v for i, e in enumerate(entries) if e.feed is not None
                         for v in (seg_start[i] + lens[i] - 1, e.feed)], dtype=np.int64)
        # "feed" comes last: recorded graphs hold the offsets of the sections before it, which for a step of
        # single tokens depend on the number of requests only
        sections = [("token_ids", token_ids), ("positions", positions), ("token_row", token_row),
                    ("seg_row", rows), ("seg_start", seg_start), ("seg_len", lens), ("seg_pos0", starts),
                    ("logit_rows", logit_rows), ("tile_info", tile_info), ("decode_info", decode_info),
                    ("big_tile_info", big_tile_info), ("rest_tile_info", rest_tile_info), ("feed", feed)]
        offsets, total = {}, 0
        for name, values in sections:
            offsets[name] = (total, len(values))
            total += _align4(max(len(values), 1))
        packed = np.zeros(total, dtype=np.int32)
        for name, values in sections:
            begin, count = offsets[name]
            packed[begin:begin + count] = values
        host = dict(seg_row=rows, seg_start=seg_start, seg_len=lens, seg_pos0=starts)
        return packed, offsets, host, n, s, int((starts + lens).max())

    def _context(self, offsets, host, n, s, max_context, min_context=0):
        def section(name):
            begin, count = offsets[name]
            return self._meta_dev[begin:begin + count]
        return StepContext(
            n_tokens=n, n_segments=s, dtype=self.model.dtype, device=self.device,
            token_ids=section("token_ids"), positions=section("positions"), token_row=section("token_row"),
            seg_row=section("seg_row"), seg_start=section("seg_start"), seg_len=section("seg_len"),
            seg_pos0=section("seg_pos0"), n_tiles=offsets["tile_info"][1] // 4, tile_info=section("tile_info"),
            n_decode=offsets["decode_info"][1] // 4, decode_info=section("decode_info"),
            n_big_tiles=offsets["big_tile_info"][1] // 4, big_tile_info=section("big_tile_info"),
            n_rest_tiles=offsets["rest_tile_info"][1] // 4, rest_tile_info=section("rest_tile_info"),
            max_context=max_context, min_context=min_context, h_seg_row=host["seg_row"], h_seg_start=host["seg_start"],
            h_seg_len=host["seg_len"], h_seg_pos0=host["seg_pos0"], extras=self._extras)

    def _upload(self, packed):
        self._reserve(len(packed))
        if self.device.type != "cuda":
            self._meta_dev[:len(packed)] = torch.from_numpy(packed)
            return
        self.last_upload_bytes = packed.nbytes
        stage = self._ring.acquire(packed.nbytes).view(torch.int32)[:len(packed)]
        stage.numpy()[:] = packed
        self._meta_dev[:len(packed)].copy_(stage, non_blocking=True)
        self._ring.commit()

    # ------------------------------------------------------------------ running
    def run(self, entries, token_source=None) -> torch.Tensor | None:
        """Run one step; float32 logits [wanted, vocab] in the order of entries and ``want``.

        Pages for the new tokens are taken first, the cache's progress moves after the
        layers have been queued.  On an exception the requests of the batch may hold
        partly written pages: the caller retires them (qil/engine.py:87-93).
        ``token_source``: int32 on the device, read on the stream for entries with ``feed``.
        """
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self._validate(entries)
        for entry in entries:
            self.cache.ensure(entry.request_id, self.cache.written(entry.request_id) + len(entry.tokens))
        packed, offsets, host, n, s, max_context = self._describe(entries)
        self.cache.flush_tables()
        self._upload(packed)
        feed_begin, feed_count = offsets["feed"]
        if feed_count:
            if token_source is None:
                raise StepError("entries with a fed token need the device buffer the tokens come from")
            begin = offsets["token_ids"][0]
            ops.feed_tokens(self._meta_dev[begin:begin + n], self._meta_dev[feed_begin:feed_begin + feed_count],
                            feed_count // 2, token_source)
        all_single = offsets["tile_info"][1] == 0 and offsets["logit_rows"][1] == n \
            and all(e.want == [0] for e in entries)
        if self.use_graphs and all_single and n <= self.graph_max_batch:
            logits = self._run_graph(offsets, host, n, s, max_context)
        else:
            ctx = self._context(offsets, host, n, s, max_context)
            begin, count = offsets["logit_rows"]
            before = ops.launch_count()
            logits = self.model.forward(ctx, self.views, self._meta_dev[begin:begin + count] if count else None)
            self.kernel_launches += ops.launch_count() - before
        for entry in entries:
            self.cache.advance(entry.request_id, self.cache.written(entry.request_id) + len(entry.tokens))
        self.steps_run += 1
        return logits

    def _run_graph(self, offsets, host, n, s, max_context):
        """Replay (after recording, the first time) the graphs of an all-single-token step.

        A step is recorded as a chain of graphs, a few layers each, not as one: submitting a graph of
        several hundred kernels takes the host most of a millisecond before the GPU sees any of it,
        and a step cannot be submitted before the previous one's tokens are known.  With a chain the
        GPU runs the first layers while the host submits the rest.
        """
        bucket = 512
        while bucket < max_context:
            bucket *= 2
        key = (n, bucket)
        record = self._graphs.get(key)
        if record is None:
            ctx = self._context(offsets, host, n, s, bucket, min_context=bucket // 2 + 1 if bucket > 512 else 1)
            begin, count = offsets["logit_rows"]
            logit_rows = self._meta_dev[begin:begin + count]
            # one eager run first: libraries set up their workspaces outside the recording
            self.model.forward(ctx, self.views, logit_rows)
            torch.cuda.synchronize()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            graphs = []
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            before = ops.launch_count()
            with torch.cuda.stream(stream):
                current = torch.cuda.CUDAGraph()
                current.capture_begin(pool=self._graph_pool)

                def cut():
                    nonlocal current
                    current.capture_end()
                    graphs.append(current)
                    current = torch.cuda.CUDAGraph()
                    current.capture_begin(pool=self._graph_pool)

                try:
                    logits = self.model.forward(ctx, self.views, logit_rows, checkpoint=cut)
                finally:
                    current.capture_end()
                graphs.append(current)
            torch.cuda.current_stream().wait_stream(stream)
            # the graphs hold addresses of what the parts keep in ``extras`` (scratch): keep those alive
            record = (graphs, logits, ops.launch_count() - before, dict(self._extras))
            self._graphs[key] = record
            self.launches_per_graph[n] = record[2]
        graphs, logits, launches = record[:3]
        for graph in graphs:
            graph.replay()
        self.kernel_launches += launches
        return logits
