"""Pinned host buffers for asynchronous host-to-device copies.

An asynchronous copy reads its pinned source when the stream reaches it, which
can be long after the Python code that queued it has moved on.  A source that the
host keeps editing (a block table, a metadata array) must therefore be
snapshotted: ``PinnedRing`` hands out one of a few pinned buffers, and takes a
buffer back only after the copies queued from it have run.
"""
from __future__ import annotations

import torch


class PinnedRing:
    def __init__(self, nbytes=1 << 16, depth=4):
        self.depth = depth
        self.buffers = [None] * depth
        self.events = [None] * depth
        self._spare = [None] * depth      # one event per buffer, made once
        self.nbytes = int(nbytes)
        self.index = 0

    def acquire(self, nbytes) -> torch.Tensor:
        """A pinned uint8 buffer of at least ``nbytes``; call ``commit`` after queueing its copies."""
        i = self.index
        if self.events[i] is not None:
            self.events[i].synchronize()
            self.events[i] = None
        if self.buffers[i] is None or self.buffers[i].numel() < nbytes:
            size = max(self.nbytes, int(nbytes))
            self.buffers[i] = torch.empty(size, dtype=torch.uint8, pin_memory=True)
        return self.buffers[i]

    def commit(self) -> None:
        event = self._spare[self.index]
        if event is None:
            event = self._spare[self.index] = torch.cuda.Event()
        event.record()
        self.events[self.index] = event
        self.index = (self.index + 1) % self.depth
