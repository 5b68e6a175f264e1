"""Host-to-device staging of a step's small index arrays.

The copy from pinned memory is asynchronous: it runs when its stream reaches it, which
may be long after the host has gone on to build the next step.  A single staging buffer
would then be overwritten before it was read (the kernels of step k would see the
arrays of step k+1).  `PinnedRing` therefore rotates over several pinned buffers and
waits on the event recorded behind a buffer's last copy before it writes to it again.

The copy across the bus runs on a stream of its own into a device-side staging buffer,
so that it happens while the step before still computes; the step's own stream then
only waits for that event and moves the arrays from the staging buffer to their place,
device to device.  (In line on the step's stream, the copy engine's turn-around stood
between two steps: some 15 us of an idle GPU.)
"""
from __future__ import annotations

import numpy as np
import torch


class PinnedRing:
    def __init__(self, device, slots: int = 4):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self._bufs = [None] * slots
        self._events = [None] * slots       # behind each pinned buffer's last copy across the bus
        self._staged = [None] * slots       # device-side staging buffers
        self._consumed = [None] * slots     # behind each staging buffer's last device-to-device copy
        self._side = None
        self._next = 0

    def send(self, host: np.ndarray, dst: torch.Tensor) -> None:
        """Copy the int32 array `host` into the front of the device tensor `dst`."""
        n = host.shape[0]
        if not self.cuda:
            dst[:n].copy_(torch.from_numpy(host))
            return
        i = self._next
        self._next = (i + 1) % len(self._bufs)
        if self._events[i] is not None:
            self._events[i].synchronize()
        buf = self._bufs[i]
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 4096), dtype=torch.int32).pin_memory()
            self._bufs[i] = buf
        buf[:n].copy_(torch.from_numpy(host))
        if self._side is None:
            self._side = torch.cuda.Stream(self.device)
        main, side = torch.cuda.current_stream(self.device), self._side
        staged = self._staged[i]
        if staged is None or staged.numel() < n:
            # Allocated under the copy stream: a block that the allocator hands out under the step's stream may
            # still be in use by kernels queued there (a tensor freed on the host while its step runs), which is
            # in order for work on that stream and a race for a copy on another one.
            with torch.cuda.stream(side):
                staged = torch.empty(max(n, 4096), dtype=torch.int32, device=self.device)
            staged.record_stream(main)
            self._staged[i] = staged
            self._consumed[i] = None
        if self._consumed[i] is not None:
            side.wait_event(self._consumed[i])          # the staging buffer's last reader is done
        with torch.cuda.stream(side):
            staged[:n].copy_(buf[:n], non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(side)
        self._events[i] = arrived
        main.wait_event(arrived)
        dst[:n].copy_(staged[:n], non_blocking=True)
        consumed = torch.cuda.Event()
        consumed.record(main)
        self._consumed[i] = consumed
