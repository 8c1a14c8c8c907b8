"""Host-to-device uploads of a step's description that may be queued ahead.

A replayed step reads its tokens, positions, lengths and page tables from
fixed device buffers that one copy from pinned memory refreshes. The copy is
asynchronous: when the host prepares steps faster than the device runs them
(device-resident decoding never waits for the device), a pinned buffer that is
rewritten for step k+1 may still be the source of step k's queued copy, and
step k would then run with step k+1's positions.

`StagingRing` therefore keeps the values in ordinary host memory (`values`)
and sends them through a ring of pinned buffers, each guarded by an event
recorded behind its copy: a buffer is rewritten only after the copy that last
read it has run. The host can be at most `depth` uploads ahead of the device.
"""
from __future__ import annotations

import numpy as np
import torch


class StagingRing:
    def __init__(self, count: int, dtype: torch.dtype, device: torch.device, depth: int = 4):
        self.dev = torch.zeros(count, dtype=dtype, device=device)
        self.values = torch.zeros(count, dtype=dtype).numpy()  # what the next upload sends
        self._pinned = [torch.zeros(count, dtype=dtype).pin_memory() for _ in range(depth)]
        self._views = [p.numpy() for p in self._pinned]
        self._events = [None] * depth
        self._next = 0

    def upload(self, start: int = 0) -> int:
        """Queue a copy of `values[start:]` to `dev[start:]` on the current
        stream; returns the bytes sent."""
        i = self._next
        self._next = (i + 1) % len(self._pinned)
        event = self._events[i]
        if event is not None:
            event.synchronize()  # the copy that last read this buffer has run
        else:
            event = self._events[i] = torch.cuda.Event()
        np.copyto(self._views[i][start:], self.values[start:])
        self.dev[start:].copy_(self._pinned[i][start:], non_blocking=True)
        event.record()
        return (self.values.size - start) * self.values.itemsize
