"""Pinned host buffers for the small per-step copies to the device.

A copy from pinned memory returns before it has run, so a buffer is written again only
after the event recorded behind its last copy has passed; a ring of buffers keeps the
host from ever waiting in practice.
"""
from __future__ import annotations

import torch


class PinnedRing:
    def __init__(self, capacity: int, depth: int = 4):
        self.capacity, self.depth = capacity, depth
        self._buffers = [torch.empty(capacity, dtype=torch.int32).pin_memory() for _ in range(depth)]
        self._arrays = [buffer.numpy() for buffer in self._buffers]
        self._events = [None] * depth
        self._next = 0

    def acquire(self, count: int):
        """A pinned int32 array of `count` elements to fill, and its ticket."""
        if count > self.capacity:
            raise ValueError(f"{count} ints exceed the staging capacity of {self.capacity}")
        ticket = self._next
        self._next = (self._next + 1) % self.depth
        if self._events[ticket] is not None:
            self._events[ticket].synchronize()
        return self._arrays[ticket][:count], ticket

    def upload(self, ticket: int, count: int, target: torch.Tensor) -> None:
        """Copies the first `count` ints of the ticket's buffer into `target[:count]` on the current stream."""
        target[:count].copy_(self._buffers[ticket][:count], non_blocking=True)
        event = self._events[ticket] or torch.cuda.Event()
        event.record()
        self._events[ticket] = event
