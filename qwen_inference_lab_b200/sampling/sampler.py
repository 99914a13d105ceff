"""Choosing next tokens from the step's logits.

Greedy: the largest logit, lowest index among equals; non-finite logits are an
error, not a token (qil/engine.py:96-100).  Temperature: a draw from
``softmax(logits / temperature)`` by the Gumbel-max rule with noise that depends
only on (the request's seed, the index of the token being drawn, the vocabulary
index), so that a request's tokens do not change with the batch it shares.
The reference samples greedily only.

Two ways to give a row its settings.  ``begin``/``choose`` with host sequences copy three small
arrays to the device per call.  The engine does not: each request's temperature, seed and number of
draws live in its state slot on the device (``SLOT``, zeroed at admission = greedy; ``configure``
writes the first two once, when a request that samples with a temperature is first seen), the
kernel finds a row's slot through ``owner`` (part of the step's one upload) and counts the draws
itself, so sampling uploads nothing per step.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..parts.base import StateSpec

#: per-request sampler state: (the temperature's float32 bits, seed, draws so far, unused)
SLOT = StateSpec((4,), torch.int64)


class NonFiniteLogits(RuntimeError):
    pass


class _Ticket:
    __slots__ = ("tokens", "host", "event", "rows")

    def __init__(self, tokens, host, event, rows):
        self.tokens, self.host, self.event, self.rows = tokens, host, event, rows


class Sampler:
    def __init__(self, device, max_rows=256):
        self.device = torch.device(device)
        self._views = {}
        self._async = [None, None]      # two sets of (device pair, pinned pair, its numpy view, event) for begin/finish
        self._next_slot = 1
        self._allocate(max_rows)

    def _allocate(self, rows):
        self._result = torch.zeros((2, rows), dtype=torch.int32, device=self.device)
        self._host = torch.zeros((2, rows), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        self._host_numpy = self._host.numpy()
        self._views.clear()

    def _reserve(self, rows):
        if rows > self._result.shape[1]:
            self._allocate(rows)

    def _buffers(self, rows):
        """(tokens, flags) on the device, the (device, host) pair of the read-back, for this row count."""
        views = self._views.get(rows)
        if views is None:
            views = (self._result[0, :rows], self._result[1, :rows], self._result[:, :rows], self._host[:, :rows])
            self._views[rows] = views
        return views

    def configure(self, state, row, temperature, seed) -> None:
        """Write a request's settings into its slot (``state`` int64 [slots, 4]); its draw count starts at 0.
        Only requests that sample with a temperature need this: a zeroed slot is greedy."""
        bits = torch.tensor([temperature], dtype=torch.float32).view(torch.int32).item()
        values = torch.tensor([bits, seed & 0x7FFFFFFFFFFFFFFF, 0, 0], dtype=torch.int64)
        if self.device.type == "cuda":
            values = values.pin_memory()
        state[row].copy_(values, non_blocking=True)

    def begin(self, logits, temperatures=None, seeds=None, counters=None, *, state=None, owner=None):
        """Queue the choice for every row of ``logits`` and its copy to the host; nothing waits.
        Settings from host sequences, or from the requests' slots (``state``, ``owner``: see the module's text).

        Returns a ticket for ``finish``; ``ticket.tokens`` is the int32 device tensor [R] that holds the
        chosen ids once the stream gets there (the next step may read it on the stream before the
        host does).  Two tickets may be open at a time: buffers alternate.
        """
        rows = logits.shape[0]
        slot = self._next_slot = (self._next_slot + 1) % 2
        pair = self._async[slot]
        if pair is None or pair[0].shape[1] < rows:
            size = max(rows, self._result.shape[1])
            device = torch.zeros((2, size), dtype=torch.int32, device=self.device)
            host = torch.zeros((2, size), dtype=torch.int32, pin_memory=self.device.type == "cuda")
            pair = self._async[slot] = (device, host, host.numpy(), torch.cuda.Event())
        device, host, host_numpy, event = pair
        t = s = c = None
        if temperatures is not None and any(v > 0 for v in temperatures):
            t = torch.tensor(list(temperatures), dtype=torch.float32).to(self.device, non_blocking=True)
            s = torch.tensor([v & 0x7FFFFFFFFFFFFFFF for v in seeds], dtype=torch.int64).to(self.device, non_blocking=True)
            c = torch.tensor(list(counters), dtype=torch.int64).to(self.device, non_blocking=True)
        tokens = device[0, :rows]
        ops.sample_rows(logits, t, s, c, tokens=tokens, nonfinite=device[1, :rows], state=state, owner=owner)
        host[:, :rows].copy_(device[:, :rows], non_blocking=True)
        event.record()
        return _Ticket(tokens, host_numpy, event, rows)

    def finish(self, ticket) -> list:
        """Wait for a ticket's copy; the chosen ids, or NonFiniteLogits."""
        ticket.event.synchronize()
        if ticket.host[1, :ticket.rows].any():
            raise NonFiniteLogits("model returned non-finite logits")
        return ticket.host[0, :ticket.rows].tolist()

    def choose(self, logits, temperatures=None, seeds=None, counters=None) -> list:
        """One token id per row of float32 ``logits`` [R, V]; waits for the result.

        ``temperatures`` (0 = greedy), ``seeds`` and ``counters`` are host sequences of
        length R, or None for an all-greedy batch.
        """
        rows = logits.shape[0]
        self._reserve(rows)
        t = s = c = None
        if temperatures is not None and any(v > 0 for v in temperatures):
            t = torch.tensor(list(temperatures), dtype=torch.float32).to(self.device, non_blocking=True)
            s = torch.tensor([v & 0x7FFFFFFFFFFFFFFF for v in seeds], dtype=torch.int64).to(self.device, non_blocking=True)
            c = torch.tensor(list(counters), dtype=torch.int64).to(self.device, non_blocking=True)
        tokens, flags, device_pair, host_pair = self._buffers(rows)
        ops.sample_rows(logits, t, s, c, tokens=tokens, nonfinite=flags)
        host_pair.copy_(device_pair, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        if self._host_numpy[1, :rows].any():
            raise NonFiniteLogits("model returned non-finite logits")
        return self._host_numpy[0, :rows].tolist()
