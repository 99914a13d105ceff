"""The inference loop: plan -> one step over the batch -> sample -> events -> release.

Surface and behaviour follow the reference's ``Engine`` (qil/engine.py:12-154):
``submit`` validates and queues, ``step`` runs one budgeted plan and returns token
events, ``cancel``/``result``/``idle``/``generate``/``close`` as there.  Unlike the
reference, which runs each prefill chunk in a forward of its own and batches only
decode tokens (qil/engine.py:59-86), a step here is one batch of everything that
was planned.  If a step fails, every request in it is retired as ``failed`` and its
pages are freed, since any of them may hold partly written pages
(qil/engine.py:87-93); requests outside the batch go on.

With ``overlap=True`` the engine runs one step ahead of the host: a step is planned and queued while
the step before it is still on the GPU, the tokens that step sampled are fed to the new one on the
device (``StepEntry.feed``), and only then does the host wait for them, append them, and retire what
finished.  The GPU never waits for the host's planning.  ``step`` then returns the events of the step
before the one it queued; a request that ended with an end-of-sequence token has by then one more
token queued, which is computed and dropped.  ``generate`` and the command line use this mode;
``Engine(...)`` defaults to the reference's behaviour (a step's own events).
"""
from __future__ import annotations

from time import perf_counter

from ..cache import CacheManager
from ..sampling import Sampler
from .scheduler import Request, Scheduler
from .step import PENDING, StepEntry, StepRunner


class Engine:
    def __init__(self, model, *, num_pages=256, page_size=16, token_budget=128, prefill_chunk=64,
                 max_active=4, clock=perf_counter, seed=0, use_graphs=True, overlap=False):
        self.model = model
        self.overlap = bool(overlap)
        self._queued = None           # the step that is on the GPU and whose tokens the host has not read
        self.clock = clock
        self.seed = int(seed)
        self.next_id = 0
        self.cache = CacheManager(model.cache_specs(), num_pages=num_pages, page_size=page_size,
                                  max_requests=max_active, max_context=model.max_positions,
                                  dtype=model.dtype, device=model.device, max_step_tokens=token_budget)
        self.scheduler = Scheduler(self.cache, token_budget=token_budget, prefill_chunk=prefill_chunk,
                                   max_active=max_active)
        self.runner = StepRunner(model, self.cache, max_step_tokens=token_budget, use_graphs=use_graphs)
        self.sampler = Sampler(model.device, max_rows=max_active)
        self.counters = dict(steps=0, tokens=0, prefill_tokens=0, decode_tokens=0)

    # the reference calls its cache ``pool`` (qil/engine.py:26)
    @property
    def pool(self):
        return self.cache

    def submit(self, prompt, *, max_new_tokens=64, ignore_eos=False, temperature=0.0, seed=None):
        prompt = list(prompt)
        vocab = self.model.vocab_size
        if not prompt or any(type(t) is not int or not 0 <= t < vocab for t in prompt):
            raise ValueError("prompt must contain valid integer token IDs")
        if type(max_new_tokens) is not int or max_new_tokens < 1:
            raise ValueError("max_new_tokens must be a positive integer")
        if len(prompt) + max_new_tokens > self.model.max_positions:
            raise ValueError("request exceeds model context length")
        if isinstance(temperature, bool) or not isinstance(temperature, (int, float)) or not temperature >= 0 \
                or temperature == float("inf"):
            raise ValueError("temperature must be a finite number >= 0")
        if seed is not None and type(seed) is not int:
            raise ValueError("seed must be an integer")
        eos = set() if ignore_eos else set(getattr(self.model.config, "eos_token_ids", ()))
        request_id = self.next_id
        request_seed = seed if seed is not None else self.seed * 1000003 + request_id
        self.scheduler.add(Request(request_id, prompt, max_new_tokens, eos, self.clock(),
                                   temperature=float(temperature), seed=request_seed))
        self.next_id += 1
        return request_id

    def step(self) -> list:
        """Run one planned batch; returns events ``dict(request_id, token_id, timestamp_s, finished)``:
        of this batch, or with ``overlap`` of the batch queued by the call before."""
        if self.overlap:
            return self._step_ahead()
        plan = self.scheduler.plan()
        try:
            queued = self._queue(plan, None)
        except Exception as error:
            self._fail(plan, error)
            raise
        return self._collect(queued) if queued is not None else []

    def _step_ahead(self) -> list:
        before = self._queued
        plan = self.scheduler.plan()
        try:
            self._queued = self._queue(plan, before)
        except Exception as error:
            self._queued = None
            if before is not None:
                self._collect(before, quiet=True)       # its tokens are kept; the error below is the news
            self._fail(plan, error)
            raise
        return self._collect(before) if before is not None else []

    def _queue(self, plan, before):
        """Queue a plan's step and the choice of its tokens; nothing waits.  ``before``: the step whose
        tokens are still on the device (requests with a pending token take it from there)."""
        if not plan:
            return None
        requests = self.scheduler.requests
        entries, ready = [], []
        for work in plan:
            request = requests[work.request_id]
            done = work.start + len(work.tokens) == request.input_length
            feed = None
            if work.tokens[-1] == PENDING:
                feed = before["slot"][request.id]
            entries.append(StepEntry(work.request_id, work.tokens, [len(work.tokens) - 1] if done else [], feed))
            if done:
                ready.append(request)
        source = before["ticket"].tokens if before is not None and before["ticket"] is not None else None
        logits = self.runner.run(entries, source)
        ticket = None
        if ready:
            ticket = self.sampler.begin(logits, [r.temperature for r in ready], [r.seed for r in ready],
                                        [len(r.output) + r.pending for r in ready])
        for work in plan:
            requests[work.request_id].computed = work.start + len(work.tokens)
        for request in ready:
            request.pending += 1          # 2 for a moment when running ahead: this step's and the one before's
        return dict(plan=plan, ready=ready, ticket=ticket, slot={r.id: i for i, r in enumerate(ready)})

    def _fail(self, plan, error):
        for work in plan:
            request = self.scheduler.requests[work.request_id]
            if request.state == "active":
                request.error = str(error)
                request.pending = 0
                self.scheduler.retire(work.request_id, "failed", "error")

    def _collect(self, queued, quiet=False) -> list:
        """Wait for a queued step's tokens; append them, retire what finished, return the events."""
        plan, ready = queued["plan"], queued["ready"]
        requests = self.scheduler.requests
        try:
            tokens = self.sampler.finish(queued["ticket"]) if queued["ticket"] is not None else []
            self.runner.check(wait=not self.overlap)     # kernels with bounded waits report through error words
        except Exception as error:
            self._fail(plan, error)
            if quiet:
                return []
            raise
        self.counters["steps"] += 1
        for work in plan:
            count = len(work.tokens)
            self.counters["tokens"] += count
            prompt_length = len(requests[work.request_id].prompt)
            self.counters["prefill_tokens" if work.start < prompt_length else "decode_tokens"] += count
        events = []
        for request, token in zip(ready, tokens):
            if request.state != "active" or not request.pending:
                continue                # cancelled, failed or finished since: the token is dropped
            observed = self.clock()
            request.pending -= 1
            request.output.append(token)
            request.token_times_s.append(observed)
            reason = "eos" if token in request.eos else (
                "length" if len(request.output) == request.max_new_tokens else None)
            if reason:
                self.scheduler.retire(request.id, "completed", reason)
            events.append(dict(request_id=request.id, token_id=token, timestamp_s=observed,
                               finished=reason is not None))
        return events

    def cancel(self, request_id) -> bool:
        return self.scheduler.retire(request_id, "cancelled", "cancelled")

    def result(self, request_id) -> dict:
        request = self.scheduler.requests[request_id]
        times = request.token_times_s
        gaps = [b - a for a, b in zip(times, times[1:])]
        return dict(
            request_id=request_id, state=request.state, finish_reason=request.finish_reason,
            error=request.error, token_ids=list(request.output),
            token_times_s=[t - request.arrival_s for t in times],
            ttft_s=times[0] - request.arrival_s if times else None,
            e2e_s=times[-1] - request.arrival_s if request.state == "completed" else None,
            tpot_s=sum(gaps) / len(gaps) if gaps else None)

    @property
    def idle(self) -> bool:
        return self.scheduler.idle and self._queued is None

    def generate(self, prompts, *, max_new_tokens=64, ignore_eos=False, temperature=0.0, seed=None) -> list:
        if not self.idle:
            raise ValueError("generate requires an idle engine; use submit/step for live requests")
        request_ids = []
        try:
            for index, prompt in enumerate(prompts):
                request_ids.append(self.submit(
                    prompt, max_new_tokens=max_new_tokens, ignore_eos=ignore_eos, temperature=temperature,
                    seed=None if seed is None else seed + index))
            ahead, self.overlap = self.overlap, True       # nobody reads the events here: run a step ahead
            try:
                while not self.idle:
                    self.step()
            finally:
                self.overlap = ahead
        except Exception:
            for request_id in request_ids:
                self.cancel(request_id)
            raise
        return [self.result(request_id) for request_id in request_ids]

    def close(self) -> None:
        for request_id in list(self.scheduler.active) + list(self.scheduler.waiting):
            self.cancel(request_id)
        if self._queued is not None:
            queued, self._queued = self._queued, None
            self._collect(queued, quiet=True)
