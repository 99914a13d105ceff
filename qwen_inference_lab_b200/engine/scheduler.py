"""Who runs next, and how much: the planner between the requests and the step function.

The policy is the reference scheduler's (qil/scheduler.py:37-103) and is what the lifecycle tests pin:

* a request that could never fit the cache is refused when it is added; the others queue in
  arrival order;
* each plan first moves queued requests into the ring of running ones while the ring has room
  (``max_active``).  Moving in reserves cache credit for everything the request will ever cache (its
  prompt and every new token but the last), which is why pages cannot run out later; a request
  whose credit cannot be had now goes to the back of the queue, so smaller ones behind it may pass;
* then the ring is served from its head under the step's token budget: up to ``prefill_chunk``
  tokens for a request still in its prompt, one token for a request that generates.  A served
  request goes to the ring's tail, one that the budget did not reach keeps its place: no starvation;
* nothing is preempted, swapped or recomputed.

The data is this engine's own.  A request is a :class:`Sequence`; the planner hands the step function
ready-made :class:`~.step.StepEntry` objects (one :class:`Turn` per served request), and it keeps the
books for running a step ahead of the host: a token that a queued step has chosen and the host has not
read yet (``unread``) already counts as input, its place in the next entry holds ``PENDING`` and names
the row of the device buffer it will be fed from.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass

from .step import PENDING, StepEntry

WAITING, ACTIVE, COMPLETED, CANCELLED, FAILED = "waiting", "active", "completed", "cancelled", "failed"


class Sequence:
    """One request from submission to its last token.

    ``fed`` counts the input tokens (prompt, then generated ones) that steps have consumed or been
    queued with; ``unread`` the generated tokens that are still on the device; ``feed_row`` where the
    latest of those sits in the sampler's device buffer.
    """

    __slots__ = ("id", "prompt", "max_new_tokens", "eos", "arrival_s", "temperature", "seed", "output",
                 "token_times_s", "fed", "unread", "feed_row", "sampler_ready", "state", "finish_reason", "error")

    def __init__(self, id, prompt, max_new_tokens, eos=(), arrival_s=0.0, *, temperature=0.0, seed=0):
        self.id, self.prompt, self.max_new_tokens = id, list(prompt), int(max_new_tokens)
        self.eos, self.arrival_s = set(eos), arrival_s
        self.temperature, self.seed = float(temperature), int(seed)
        self.output, self.token_times_s = [], []
        self.fed = self.unread = 0
        self.feed_row = None
        self.sampler_ready = False
        self.state, self.finish_reason, self.error = WAITING, None, None

    def __repr__(self):
        return f"Sequence({self.id}, {self.state}, fed {self.fed} of {self.input_length})"

    @property
    def known_length(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def input_length(self) -> int:
        """Tokens that can be fed now: the known ones and those still on the device."""
        return self.known_length + self.unread

    @property
    def in_prompt(self) -> bool:
        return self.fed < len(self.prompt)

    @property
    def reservation(self) -> int:
        """Positions this request will ever cache: its last new token is returned, never fed
        (qil/scheduler.py:24-27)."""
        return len(self.prompt) + self.max_new_tokens - 1

    @property
    def awaits_last_token(self) -> bool:
        """All its tokens are chosen, the last of them unread: there is nothing left to feed."""
        return self.unread > 0 and len(self.output) + self.unread >= self.max_new_tokens

    def tokens_from(self, start, count) -> list:
        """Input tokens [start, start + count) without building the whole input; PENDING where the
        token is still on the device."""
        split, known = len(self.prompt), self.known_length
        taken = self.prompt[start:start + count] if start < split else []
        if len(taken) < count and start + count > split:
            lo = max(start, split) - split
            taken = taken + self.output[lo:lo + count - len(taken)]
        return taken + [PENDING] * (start + count - max(start, known)) if start + count > known else taken

    def report(self) -> dict:
        """What ``Engine.result`` returns (fields and meanings of qil/engine.py:120-131)."""
        since_arrival = [stamp - self.arrival_s for stamp in self.token_times_s]
        several = len(since_arrival) > 1
        return {
            "request_id": self.id, "state": self.state, "finish_reason": self.finish_reason, "error": self.error,
            "token_ids": list(self.output), "token_times_s": since_arrival,
            "ttft_s": since_arrival[0] if since_arrival else None,
            "e2e_s": since_arrival[-1] if self.state == COMPLETED and since_arrival else None,
            "tpot_s": (since_arrival[-1] - since_arrival[0]) / (len(since_arrival) - 1) if several else None,
        }


@dataclass
class Turn:
    """One request's share of a planned step."""
    sequence: Sequence
    start: int               # position of the entry's first token
    entry: StepEntry

    @property
    def samples(self) -> bool:
        """The entry ends the request's input: the step chooses its next token."""
        return bool(self.entry.want)

    @property
    def count(self) -> int:
        return len(self.entry.tokens)


class Scheduler:
    def __init__(self, cache, *, token_budget=128, prefill_chunk=64, max_active=4):
        for name, value in (("token_budget", token_budget), ("prefill_chunk", prefill_chunk), ("max_active", max_active)):
            if type(value) is not int or value < 1:
                raise ValueError(f"{name} must be a positive integer, got {value!r}")
        self.cache = cache
        self.token_budget, self.prefill_chunk, self.max_active = token_budget, prefill_chunk, max_active
        self.table: dict = {}              # id -> Sequence, finished ones included
        self.queue: deque = deque()        # waiting, in arrival order (re-queued ones at the back)
        self.ring: deque = deque()         # active; the next to be served is at the left

    # ------------------------------------------------------------------ arrivals
    def add(self, sequence) -> None:
        if sequence.id in self.table:
            raise ValueError(f"request id {sequence.id!r} is already in use (duplicate)")
        if not self.cache.fits(sequence.reservation):
            raise ValueError(f"a request of {sequence.reservation} cached tokens exceeds the cache's capacity: "
                             f"shorten it or give the engine more pages")
        self.table[sequence.id] = sequence
        self.queue.append(sequence)

    def _admit(self) -> None:
        for _ in range(len(self.queue)):
            if len(self.ring) >= self.max_active:
                return
            sequence = self.queue.popleft()
            if self.cache.admit(sequence.id, sequence.reservation):
                sequence.state = ACTIVE
                self.ring.append(sequence)
            else:
                self.queue.append(sequence)

    # ------------------------------------------------------------------ planning
    def plan(self) -> list:
        """The next step as a list of turns (possibly empty: everybody waits for a last token)."""
        self._admit()
        turns, room = [], self.token_budget
        for _ in range(len(self.ring)):
            if room == 0:
                break
            sequence = self.ring[0]
            self.ring.rotate(-1)                       # served, or waiting for its last token: to the tail
            if sequence.awaits_last_token:
                continue
            share = self.prefill_chunk if sequence.in_prompt else 1
            count = min(share, room, sequence.input_length - sequence.fed)
            if count < 1:
                raise RuntimeError(f"request {sequence.id!r} is active with nothing left to feed")
            turns.append(self._turn(sequence, count))
            room -= count
        if not turns and self.queue and not self.ring:
            raise RuntimeError("requests are waiting, none is active and none could be admitted")
        return turns

    @staticmethod
    def _turn(sequence, count) -> Turn:
        start = sequence.fed
        tokens = sequence.tokens_from(start, count)
        ends_input = start + count == sequence.input_length
        feed = sequence.feed_row if tokens[-1] == PENDING else None
        return Turn(sequence, start, StepEntry(sequence.id, tokens, [count - 1] if ends_input else [], feed))

    def queued(self, turns) -> None:
        """The turns have been handed to the step function: their tokens count as fed, and each turn that
        samples leaves one more token on the device, in the row it has among the sampling turns."""
        row = 0
        for turn in turns:
            sequence = turn.sequence
            sequence.fed = turn.start + turn.count
            if turn.samples:
                sequence.unread += 1               # two for a moment when running ahead: this step's and the last's
                sequence.feed_row = row
                row += 1

    def read(self, sequence, token, now):
        """A token has arrived on the host.  None if the sequence no longer takes tokens (cancelled, failed,
        or finished on an earlier token: the token is dropped), else the event of qil/engine.py:114-115."""
        if sequence.state != ACTIVE or not sequence.unread:
            return None
        sequence.unread -= 1
        sequence.output.append(token)
        sequence.token_times_s.append(now)
        if token in sequence.eos:                       # checked first: an end token at full length is "eos"
            reason = "eos"
        elif len(sequence.output) >= sequence.max_new_tokens:
            reason = "length"
        else:
            reason = None
        if reason is not None:
            self.retire(sequence.id, COMPLETED, reason)
        return {"request_id": sequence.id, "token_id": token, "timestamp_s": now, "finished": reason is not None}

    # ------------------------------------------------------------------ endings
    def retire(self, request_id, state, reason) -> bool:
        """Take a waiting or active request out (False if it has ended before); an active one frees its cache."""
        sequence = self.table[request_id]
        if sequence.state == WAITING:
            self.queue.remove(sequence)
        elif sequence.state == ACTIVE:
            self.ring.remove(sequence)
            self.cache.release(request_id)
        else:
            return False
        sequence.state, sequence.finish_reason, sequence.unread = state, reason, 0
        return True

    @property
    def idle(self) -> bool:
        return not (self.queue or self.ring)

    @property
    def prefilling(self) -> bool:
        """Is any request that has not ended still in its prompt?"""
        return any(s.in_prompt for s in self.queue) or any(s.in_prompt for s in self.ring)
