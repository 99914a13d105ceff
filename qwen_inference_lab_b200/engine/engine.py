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
from ..sampling import SLOT, Sampler
from .scheduler import ACTIVE, Scheduler, Sequence
from .step import StepRunner


class _Flight:
    """A step that has been queued on the GPU: its turns, the sequences it chooses tokens for (in the order
    of the sampler's rows) and the sampler's ticket for them."""
    __slots__ = ("turns", "sampling", "ticket")

    def __init__(self, turns, sampling, ticket):
        self.turns, self.sampling, self.ticket = turns, sampling, ticket


class Engine:
    def __init__(self, model, *, num_pages=256, page_size=16, token_budget=128, prefill_chunk=64,
                 max_active=4, clock=perf_counter, seed=0, use_graphs=True, overlap=False):
        self.model = model
        self.overlap = bool(overlap)
        self.clock = clock
        self.seed = int(seed)
        self.next_id = 0
        self._in_flight = None        # the step that is on the GPU and whose tokens the host has not read
        self.cache = CacheManager(model.cache_specs(), num_pages=num_pages, page_size=page_size,
                                  max_requests=max_active, max_context=model.max_positions,
                                  dtype=model.dtype, device=model.device, max_step_tokens=token_budget,
                                  request_state={"sampler": SLOT})
        self.scheduler = Scheduler(self.cache, token_budget=token_budget, prefill_chunk=prefill_chunk,
                                   max_active=max_active)
        self.runner = StepRunner(model, self.cache, max_step_tokens=token_budget, use_graphs=use_graphs)
        self.sampler = Sampler(model.device, max_rows=max_active)
        self.counters = dict(steps=0, tokens=0, prefill_tokens=0, decode_tokens=0)

    # the reference calls its cache ``pool`` (qil/engine.py:26)
    @property
    def pool(self):
        return self.cache

    # ------------------------------------------------------------------ requests in
    def _check_submission(self, prompt, max_new_tokens, temperature, seed) -> None:
        """The reference's three checks (qil/engine.py:35-40), then the sampling settings."""
        vocab = self.model.vocab_size
        if len(prompt) == 0:
            raise ValueError("the prompt is empty; it must hold at least one token id")
        for token in prompt:
            if type(token) is not int or token < 0 or token >= vocab:
                raise ValueError(f"the prompt holds {token!r}; token ids must be integers in [0, {vocab})")
        if type(max_new_tokens) is not int or max_new_tokens <= 0:
            raise ValueError(f"max_new_tokens must be a positive integer, got {max_new_tokens!r}")
        room = self.model.max_positions
        if len(prompt) + max_new_tokens > room:
            raise ValueError(f"{len(prompt)} prompt tokens and {max_new_tokens} new ones exceed the model's "
                             f"context length of {room} positions")
        number = isinstance(temperature, (int, float)) and not isinstance(temperature, bool)
        if not number or not 0 <= temperature < float("inf"):
            raise ValueError("temperature must be a finite number >= 0")
        if seed is not None and type(seed) is not int:
            raise ValueError("seed must be an integer")

    def submit(self, prompt, *, max_new_tokens=64, ignore_eos=False, temperature=0.0, seed=None):
        prompt = list(prompt)
        self._check_submission(prompt, max_new_tokens, temperature, seed)
        stops = () if ignore_eos else getattr(self.model.config, "eos_token_ids", ())
        request_id = self.next_id
        if seed is None:
            seed = self.seed * 1000003 + request_id
        self.scheduler.add(Sequence(request_id, prompt, max_new_tokens, stops, self.clock(),
                                    temperature=temperature, seed=seed))
        self.next_id = request_id + 1
        return request_id

    # ------------------------------------------------------------------ steps
    def step(self) -> list:
        """Run one planned batch; returns events ``dict(request_id, token_id, timestamp_s, finished)``:
        of this batch, or with ``overlap`` of the batch queued by the call before."""
        earlier = self._in_flight if self.overlap else None
        turns = self.scheduler.plan()
        try:
            flight = self._launch(turns, earlier)
        except Exception as error:
            self._in_flight = None
            if earlier is not None:
                self._land(earlier, quiet=True)        # its tokens are kept; the error below is the news
            self._fail(turns, error)
            raise
        if self.overlap:
            self._in_flight = flight
            return self._land(earlier) if earlier is not None else []
        return self._land(flight) if flight is not None else []

    def _launch(self, turns, earlier):
        """Queue a plan's step and the choice of its tokens; nothing waits.  ``earlier``: the step whose
        tokens are still on the device (entries with a pending token take it from there)."""
        if not turns:
            return None
        source = earlier.ticket.tokens if earlier is not None and earlier.ticket is not None else None
        logits = self.runner.run([turn.entry for turn in turns], source)
        sampling = [turn.sequence for turn in turns if turn.samples]
        ticket = None
        if sampling:
            state = self.cache.request_state("sampler")
            for sequence in sampling:
                if sequence.temperature > 0 and not sequence.sampler_ready:
                    self.sampler.configure(state, self.cache.row(sequence.id), sequence.temperature, sequence.seed)
                    sequence.sampler_ready = True
            ticket = self.sampler.begin(logits, state=state, owner=self.runner.logit_owner)
        self.scheduler.queued(turns)
        return _Flight(turns, sampling, ticket)

    def _fail(self, turns, error) -> None:
        """A step that failed may have left any of its requests with partly written pages: all of them end
        as failed and free their cache; requests outside the batch go on (qil/engine.py:87-93)."""
        for turn in turns:
            if turn.sequence.state == ACTIVE:
                turn.sequence.error = str(error)
                self.scheduler.retire(turn.sequence.id, "failed", "error")

    def _land(self, flight, quiet=False) -> list:
        """Wait for a queued step's tokens; append them, retire what finished, return the events."""
        try:
            tokens = self.sampler.finish(flight.ticket) if flight.ticket is not None else []
            self.runner.check(wait=not self.overlap)     # kernels with bounded waits report through error words
        except Exception as error:
            self._fail(flight.turns, error)
            if quiet:
                return []
            raise
        counters = self.counters
        counters["steps"] += 1
        for turn in flight.turns:
            counters["tokens"] += turn.count
            counters["prefill_tokens" if turn.start < len(turn.sequence.prompt) else "decode_tokens"] += turn.count
        events = []
        for sequence, token in zip(flight.sampling, tokens):
            event = self.scheduler.read(sequence, token, self.clock())
            if event is not None:
                events.append(event)
        return events

    # ------------------------------------------------------------------ requests out
    def cancel(self, request_id) -> bool:
        return self.scheduler.retire(request_id, "cancelled", "cancelled")

    def result(self, request_id) -> dict:
        return self.scheduler.table[request_id].report()

    @property
    def idle(self) -> bool:
        return self._in_flight is None and self.scheduler.idle

    def generate(self, prompts, *, max_new_tokens=64, ignore_eos=False, temperature=0.0, seed=None) -> list:
        """Submit all prompts, step until nothing is left, return their results in order.  Runs a step ahead
        of the host (nobody reads the events here).  On an error every request of the call is cancelled."""
        if not self.idle:
            raise ValueError("generate() needs an idle engine; feed a busy one with submit() and step()")
        mine = []
        mode, self.overlap = self.overlap, True
        try:
            for index, prompt in enumerate(prompts):
                mine.append(self.submit(prompt, max_new_tokens=max_new_tokens, ignore_eos=ignore_eos,
                                        temperature=temperature, seed=seed if seed is None else seed + index))
            while not self.idle:
                self.step()
        except Exception:
            for request_id in mine:
                self.cancel(request_id)
            raise
        finally:
            self.overlap = mode
        return [self.result(request_id) for request_id in mine]

    def close(self) -> None:
        """Cancel whatever has not ended and wait for the step that may still be on the GPU."""
        for sequence in [*self.scheduler.ring, *self.scheduler.queue]:
            self.cancel(sequence.id)
        flight, self._in_flight = self._in_flight, None
        if flight is not None:
            self._land(flight, quiet=True)
