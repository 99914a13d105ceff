"""Round-robin planning of token work under a budget, with admission by reservation.

Policy of the reference's scheduler (qil/scheduler.py:37-103):

* ``add`` refuses a request that could never fit the cache; others wait in arrival order.
* every ``plan`` first admits waiting requests while fewer than ``max_active`` are
  active; admission reserves cache credit for the whole request (prompt plus all new
  tokens but the last), so pages can never run out in mid-flight; a request that
  does not fit *now* goes to the back of the waiting queue and smaller ones behind it
  may overtake.
* then the active requests take turns: a request still in its prompt gets up to
  ``prefill_chunk`` tokens, a decoding request exactly one, until ``token_budget``
  tokens are planned.  Whoever was served moves to the back; whoever was not reached
  stays in front, so nobody starves.
* there is no preemption, no swapping and no recomputation: what happens when pages
  run out is that nothing new is admitted until a request finishes and frees its own.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field


@dataclass
class Request:
    """State of one request (qil/scheduler.py:6-27), plus its sampling settings."""
    id: int
    prompt: list
    max_new_tokens: int
    eos: set
    arrival_s: float
    temperature: float = 0.0
    seed: int = 0
    output: list = field(default_factory=list)
    token_times_s: list = field(default_factory=list)
    computed: int = 0
    # output tokens that queued steps have sampled and the host has not read yet: they count as input
    # already, so the next step can be planned and queued before they are known (at most one while a
    # step is planned)
    pending: int = 0
    state: str = "waiting"            # waiting, active, completed, cancelled, failed
    finish_reason: str | None = None
    error: str | None = None

    @property
    def input_tokens(self):
        return self.prompt + self.output

    @property
    def input_length(self):
        return len(self.prompt) + len(self.output) + self.pending

    def input_slice(self, start, count):
        """``input_tokens[start:start + count]`` without building the whole list; a pending token's
        place holds PENDING (-1)."""
        split = len(self.prompt)
        known = split + len(self.output)
        if start + count > known:           # reaches into the pending token
            head = self.input_slice(start, known - start) if start < known else []
            return head + [-1] * (start + count - max(start, known))
        if start >= split:
            return self.output[start - split:start - split + count]
        if start + count <= split:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.output[:start + count - split]

    @property
    def ends_with_pending(self):
        """The pending token is the request's last: it needs no further step."""
        return self.pending > 0 and len(self.output) + self.pending >= self.max_new_tokens

    @property
    def cache_limit(self):
        # the last generated token is returned without being fed back (qil/scheduler.py:24-27)
        return len(self.prompt) + self.max_new_tokens - 1


@dataclass(frozen=True)
class Work:
    request_id: int
    start: int
    tokens: list


class Scheduler:
    def __init__(self, cache, *, token_budget=128, prefill_chunk=64, max_active=4):
        if any(type(n) is not int or n < 1 for n in (token_budget, prefill_chunk, max_active)):
            raise ValueError("scheduler budgets must be positive integers")
        self.cache = cache
        self.token_budget, self.prefill_chunk, self.max_active = token_budget, prefill_chunk, max_active
        self.requests: dict = {}
        self.waiting: deque = deque()
        self.active: deque = deque()

    def add(self, request) -> None:
        if request.id in self.requests:
            raise ValueError("duplicate request ID")
        if not self.cache.fits(request.cache_limit):
            raise ValueError("request exceeds total KV capacity; reduce tokens or increase pages")
        self.requests[request.id] = request
        self.waiting.append(request.id)

    def plan(self) -> list:
        for _ in range(len(self.waiting)):
            if len(self.active) >= self.max_active:
                break
            request_id = self.waiting.popleft()
            request = self.requests[request_id]
            if self.cache.admit(request_id, request.cache_limit):
                request.state = "active"
                self.active.append(request_id)
            else:
                self.waiting.append(request_id)
        remaining = self.token_budget
        work = []
        for _ in range(len(self.active)):
            if not remaining:
                break
            request_id = self.active.popleft()
            request = self.requests[request_id]
            if request.ends_with_pending:
                self.active.append(request_id)      # retires when its last token has been read
                continue
            chunk = self.prefill_chunk if request.computed < len(request.prompt) else 1
            count = min(chunk, remaining, request.input_length - request.computed)
            if count <= 0:
                raise RuntimeError("active request has no input to compute")
            work.append(Work(request_id, request.computed, request.input_slice(request.computed, count)))
            remaining -= count
            self.active.append(request_id)
        if not work and self.waiting and not self.active:
            raise RuntimeError("no runnable request despite an empty active set")
        return work

    def retire(self, request_id, state, reason) -> bool:
        request = self.requests[request_id]
        if request.state not in ("waiting", "active"):
            return False
        if request_id in self.waiting:
            self.waiting.remove(request_id)
        if request_id in self.active:
            self.active.remove(request_id)
            self.cache.release(request_id)
        request.state, request.finish_reason = state, reason
        return True

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.active
