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

from ctypes import byref, c_longlong, c_void_p

import numpy as np
import torch


def _check(status: int, what: str) -> None:
    if status:
        from ..kernels.ops import KernelError
        raise KernelError(f"{what} failed with status {status}" + (f" (CUDA error {status - 1000})" if status >= 1000 else ""))


def new_event(lib) -> c_void_p:
    """An event without timing from the staging library (`load_family("staging")`)."""
    ev = c_void_p()
    _check(lib.wllm_event_create(byref(ev)), "event creation")
    return ev


def free_events(lib, events) -> None:
    """Hand events back (at the end of their owner's life; an event still in use is freed when its work is done)."""
    for ev in events:
        if lib is not None and ev is not None:
            try:
                lib.wllm_event_destroy(ev)
            except Exception:       # the interpreter or the CUDA context is already going away
                pass


class PinnedRing:
    def __init__(self, device, slots: int = 4):
        self.device = torch.device(device)
        self._bufs = [None] * slots         # pinned tensors and numpy views of them
        self._views = [None] * slots
        self._staged = [None] * slots       # device-side staging buffers
        self._arrived = [None] * slots      # behind each pinned buffer's last copy across the bus
        self._consumed = [None] * slots     # behind each staging buffer's last device-to-device copy
        self._used = [False] * slots
        self._side = self._side_raw = None
        self._lib = None
        self._next = 0

    def __del__(self):
        free_events(self._lib, self._arrived + self._consumed)

    def send(self, host: np.ndarray, dst: torch.Tensor) -> None:
        """Copy the int32 array `host` into the front of the device tensor `dst`."""
        n = host.shape[0]
        if self._lib is None:
            from ..kernels.build import load_family
            self._lib = load_family("staging")
            self._side = torch.cuda.Stream(self.device)
            self._side_raw = c_void_p(self._side.cuda_stream)
        lib, i = self._lib, self._next
        self._next = (i + 1) % len(self._bufs)
        if self._arrived[i] is None:
            self._arrived[i], self._consumed[i] = new_event(lib), new_event(lib)
        elif self._used[i]:
            _check(lib.wllm_event_wait(self._arrived[i]), "waiting for a staging copy")     # the pinned buffer is free again
        if self._bufs[i] is None or self._bufs[i].numel() < n:
            self._bufs[i] = torch.empty(max(n, 4096), dtype=torch.int32).pin_memory()
            self._views[i] = self._bufs[i].numpy()
        self._views[i][:n] = host
        from ..kernels.ops import _stream
        staged, fresh = self._staged[i], False
        if staged is None or staged.numel() < n:
            # Allocated under the copy stream: a block that the allocator hands out under the step's stream may
            # still be in use by kernels queued there (a tensor freed on the host while its step runs), which is
            # in order for work on that stream and a race for a copy on another one.
            with torch.cuda.stream(self._side):
                staged = torch.empty(max(n, 4096), dtype=torch.int32, device=self.device)
            staged.record_stream(torch.cuda.current_stream(self.device))
            self._staged[i], fresh = staged, True
        _check(lib.wllm_stage_send(c_void_p(self._bufs[i].data_ptr()), c_void_p(staged.data_ptr()), c_void_p(dst.data_ptr()),
                                   c_longlong(4 * n), self._side_raw, _stream(),
                                   self._arrived[i], self._consumed[i], int(self._used[i] and not fresh)), "staging copy")
        self._used[i] = True
