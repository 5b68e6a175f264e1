"""Host-to-device staging of a step's small index arrays.

The copy from pinned memory is asynchronous: it runs when the stream reaches it, which
may be long after the host has gone on to build the next step.  A single staging buffer
would then be overwritten before it was read (the kernels of step k would see the
arrays of step k+1).  `PinnedRing` therefore rotates over several pinned buffers and
waits on the event recorded behind a buffer's last copy before it writes to it again.
"""
from __future__ import annotations

import numpy as np
import torch


class PinnedRing:
    def __init__(self, device, slots: int = 4):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self._bufs = [None] * slots
        self._events = [None] * slots
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
        dst[:n].copy_(buf[:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._events[i] = ev
