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
from ..parts.base import PlanView, Segments, StepContext
from ..utils.staging import PinnedRing


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


@dataclass
class _Description:
    """A step as it is uploaded: one int32 vector, where its sections lie, and the host's view."""
    packed: np.ndarray
    offsets: dict            # section name -> (first int, count); planners' sections are "key.name"
    segments: Segments
    max_context: int


class StepRunner:
    def __init__(self, model, cache, *, max_step_tokens=4096, use_graphs=True, graph_max_batch=256):
        self.model, self.cache = model, cache
        self.device = model.device
        self.views = cache.views(model.order)
        self.use_graphs = bool(use_graphs) and self.device.type == "cuda" and model.is_graph_safe()
        self.graph_max_batch = graph_max_batch
        planners = model.step_planners() if hasattr(model, "step_planners") else {}
        self.planners = [planners[key] for key in sorted(planners)]
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
        # the request row behind each row of the logits that the last ``run`` returned (int32, on the device;
        # valid until the next ``run`` uploads its description)
        self.logit_owner = None

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

    def _describe(self, entries) -> _Description:
        """Host arrays of the batch, packed into one int32 vector with section offsets."""
        if all(len(e.tokens) == 1 for e in entries):
            return self._describe_single_tokens(entries)
        return self._describe_general(entries)

    def _describe_single_tokens(self, entries) -> _Description:
        """The description of a step in which every request brings one token.  Consecutive decode steps
        of the same requests differ only in the tokens and the positions: the packed vector of the last
        such step is kept and those entries are overwritten.

        What is kept holds block-table rows, so the rows are part of the key: a request id that was
        released and admitted again sits in another row, and the step must be described anew.
        """
        cache = self.cache
        key = tuple((e.request_id, cache.row(e.request_id), tuple(e.want), e.feed) for e in entries)
        kept = self._single_token_template
        if kept is None or kept[0] != key:
            description = self._describe_general(entries)
            self._single_token_template = (key, description)
            return description
        description = kept[1]
        packed, offsets, segments = description.packed, description.offsets, description.segments
        n = len(entries)
        starts = np.fromiter((cache.written(e.request_id) for e in entries), dtype=np.int64, count=n)
        begin = offsets["token_ids"][0]
        packed[begin:begin + n] = [e.tokens[0] for e in entries]
        for name in ("positions", "seg_pos0"):
            begin = offsets[name][0]
            packed[begin:begin + n] = starts
        segments = Segments(rows=segments.rows, first=segments.first, lens=segments.lens, starts=starts, n_tokens=n)
        for planner in self.planners:
            arrays = {name[len(planner.key) + 1:]: packed[begin:begin + count]
                      for name, (begin, count) in offsets.items() if name.startswith(planner.key + ".")}
            if not planner.refresh_single_tokens(arrays, segments):
                description = self._describe_general(entries)
                self._single_token_template = (key, description)
                return description
        description = _Description(packed, offsets, segments, int(starts.max()) + 1)
        self._single_token_template = (key, description)
        return description

    def _describe_general(self, entries) -> _Description:
        cache = self.cache
        lens = np.array([len(e.tokens) for e in entries], dtype=np.int64)
        starts = np.array([cache.written(e.request_id) for e in entries], dtype=np.int64)
        rows = np.array([cache.row(e.request_id) for e in entries], dtype=np.int64)
        n, s = int(lens.sum()), len(entries)
        first = np.zeros(s, dtype=np.int64)
        np.cumsum(lens[:-1], out=first[1:])
        segments = Segments(rows=rows, first=first, lens=lens, starts=starts, n_tokens=n)
        token_ids = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=n)
        seg_of_token = np.repeat(np.arange(s), lens)
        positions = np.arange(n) - first[seg_of_token] + starts[seg_of_token]
        token_row = rows[seg_of_token]
        logit_rows = np.array([first[i] + w for i, e in enumerate(entries) for w in e.want], dtype=np.int64)
        logit_owner = np.array([rows[i] for i, e in enumerate(entries) for _ in e.want], dtype=np.int64)
        # places of tokens that are still on the device: (index in the flat batch, index in the source buffer)
        feed = np.array([v for i, e in enumerate(entries) if e.feed is not None
                         for v in (first[i] + lens[i] - 1, e.feed)], dtype=np.int64)
        sections = [("token_ids", token_ids), ("positions", positions), ("token_row", token_row),
                    ("seg_row", rows), ("seg_start", first), ("seg_len", lens), ("seg_pos0", starts),
                    ("logit_rows", logit_rows), ("logit_owner", logit_owner)]
        for planner in self.planners:
            for name, values in planner.plan(segments).items():
                sections.append((f"{planner.key}.{name}", np.asarray(values).reshape(-1)))
        # "feed" comes last: recorded graphs hold the offsets of the sections before it, which for a step of
        # single tokens depend on the number of requests only
        sections.append(("feed", feed))
        offsets, total = {}, 0
        for name, values in sections:
            offsets[name] = (total, len(values))
            total += _align4(max(len(values), 1))
        packed = np.zeros(total, dtype=np.int32)
        for name, values in sections:
            begin, count = offsets[name]
            packed[begin:begin + count] = values
        return _Description(packed, offsets, segments, int((starts + lens).max()))

    def _context(self, description, max_context=None, min_context=0):
        offsets, segments = description.offsets, description.segments

        def section(name):
            begin, count = offsets[name]
            return self._meta_dev[begin:begin + count]

        plans = {}
        for planner in self.planners:
            view = plans[planner.key] = PlanView()
            for name, (begin, count) in offsets.items():
                if name.startswith(planner.key + "."):
                    short = name[len(planner.key) + 1:]
                    view.array[short], view.count[short] = self._meta_dev[begin:begin + count], count
        return StepContext(
            n_tokens=segments.n_tokens, n_segments=segments.n_segments, dtype=self.model.dtype, device=self.device,
            token_ids=section("token_ids"), positions=section("positions"), token_row=section("token_row"),
            seg_row=section("seg_row"), seg_start=section("seg_start"), seg_len=section("seg_len"),
            seg_pos0=section("seg_pos0"), plans=plans,
            max_context=description.max_context if max_context is None else max_context, min_context=min_context,
            h_seg_row=segments.rows, h_seg_start=segments.first, h_seg_len=segments.lens,
            h_seg_pos0=segments.starts, extras=self._extras)

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
        description = self._describe(entries)
        offsets, n = description.offsets, description.segments.n_tokens
        self.cache.flush_tables()
        self._upload(description.packed)
        begin, count = offsets["logit_owner"]
        self.logit_owner = self._meta_dev[begin:begin + count]
        feed_begin, feed_count = offsets["feed"]
        if feed_count:
            if token_source is None:
                raise StepError("entries with a fed token need the device buffer the tokens come from")
            begin = offsets["token_ids"][0]
            ops.feed_tokens(self._meta_dev[begin:begin + n], self._meta_dev[feed_begin:feed_begin + feed_count],
                            feed_count // 2, token_source)
        all_single = all(len(e.tokens) == 1 and e.want == [0] for e in entries)
        if self.use_graphs and all_single and n <= self.graph_max_batch:
            logits = self._run_graph(description)
        else:
            ctx = self._context(description)
            begin, count = offsets["logit_rows"]
            before = ops.launch_count()
            logits = self.model.forward(ctx, self.views, self._meta_dev[begin:begin + count] if count else None)
            self.kernel_launches += ops.launch_count() - before
        for entry in entries:
            self.cache.advance(entry.request_id, self.cache.written(entry.request_id) + len(entry.tokens))
        self.steps_run += 1
        return logits

    def check(self, wait=True) -> None:
        """Raise if a kernel of an earlier step reported a fault of its own (a bounded wait that ran
        out).  Kernels with such reports register them with ``ops.register_post_step_check``.  A check
        costs nothing unless its kernel was launched since the last one; then it waits for the device,
        or with ``wait=False`` reports a step or two late instead (``ops.ErrorWord``)."""
        ops.run_post_step_checks(wait)

    def _run_graph(self, description):
        """Replay the graphs of an all-single-token step; the first step of its kind records them.

        A step is recorded as a chain of graphs, a few layers each, not as one: submitting a graph of
        several hundred kernels takes the host most of a millisecond before the GPU sees any of it,
        and a step cannot be submitted before the previous one's tokens are known.  With a chain the
        GPU runs the first layers while the host submits the rest.

        The recording step runs the model once, eagerly, outside the recording (libraries set up their
        workspaces then) and returns that run's logits; it is not replayed as well, so a part that
        updates memory in place advances once per step here too.
        """
        n = description.segments.n_tokens
        bucket = 512
        while bucket < description.max_context:
            bucket *= 2
        key = (n, bucket)
        record = self._graphs.get(key)
        if record is None:
            ctx = self._context(description, bucket, min_context=bucket // 2 + 1 if bucket > 512 else 1)
            begin, count = description.offsets["logit_rows"]
            logit_rows = self._meta_dev[begin:begin + count]
            before = ops.launch_count()
            eager_logits = self.model.forward(ctx, self.views, logit_rows)
            launches = ops.launch_count() - before
            torch.cuda.synchronize()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            graphs = []
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
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
            self._graphs[key] = (graphs, logits, launches, dict(self._extras))
            self.launches_per_graph[n] = launches
            self.kernel_launches += launches
            return eager_logits
        graphs, logits, launches = record[:3]
        for graph in graphs:
            graph.replay()
        self.kernel_launches += launches
        return logits
