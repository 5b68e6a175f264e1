"""Runs the sampling kernels over the logits rows of a step.

All rows go through the same two to five passes (statistics; up to three selection passes
when some row asks for top-k, top-p or min-p; the draw), each one launch over all rows.
Per-row options, seeds, counters and the distinct generated ids (for the repetition
penalty) travel in one int32 buffer; tokens and log-probabilities come back in one small
copy.  A batch of greedy rows without a penalty sends nothing and runs the first pass
alone.  The logits rows are modified in place where a repetition penalty applies.
"""
from __future__ import annotations

from ctypes import byref, c_int, c_longlong, c_void_p

import numpy as np
import torch

from ..kernels import ops
from ..kernels.build import load_family
from ..engine.staging import PinnedRing, free_events, new_event


class PendingSample:
    """The sampling of one step, enqueued: its tokens lie on the device (`tokens_device`, valid until the
    sampler's next launch) and are on their way to pinned host memory; `get()` waits for them."""

    def __init__(self, rows: int, tokens_device, host, done, lib, owner=None):
        self.rows, self.tokens_device, self._host, self._done, self._lib = rows, tokens_device, host, done, lib
        self._owner = owner          # the sampler (and with it the event) lives as long as its results are awaited

    def get(self):
        """(tokens, log-probabilities).  The kernels' status word came along with them: if a bounded wait in one
        of the step's kernels ran out, its results are partial, and the tokens are not handed on."""
        if self.rows == 0:
            return [], []
        ops._check(self._lib.wllm_event_wait(self._done), "waiting for the sampled ids")
        status = int(self._host[2 * self.rows])
        if status != 0:
            ops.reset_kernel_status(self._owner.device)
            raise ops.KernelError(f"a kernel of this step gave up waiting (status {status}: "
                                  f"{ops.GAVE_UP.get(status, 'unknown role')}); its tokens are not used")
        out = self._host[:2 * self.rows]
        return out[:self.rows].tolist(), out[self.rows:].view(np.float32).tolist()


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._ring = PinnedRing(self.device)
        self._dev = self._out = None
        self._out_hosts = [None, None]   # two pinned result buffers: one is read while the next step fills the other
        self._turn = 0
        self._side = self._side_raw = self._staging = None      # the results travel to the host on a stream of their own
        self._read = None                # behind the last copy out of `_out`: the next launch overwrites it
        self._scratch = None             # per-row state, chunk statistics and histograms; zero before first use
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def __del__(self):
        if self._staging is not None:
            free_events(self._staging, [self._queued] + self._done)

    def sample(self, logits: torch.Tensor, params: list, counters: list, seeds: list, generated: list):
        """logits [rows, vocab] float32 on the device; params[i]: SamplingParams; counters[i]: index of
        the output token being drawn; seeds[i]: the request's 64-bit seed; generated[i]: its distinct
        generated ids (read only when its repetition penalty is not 1).  Returns (tokens, logprobs) lists."""
        return self.sample_pending(logits, params, counters, seeds, generated).get()

    def sample_pending(self, logits: torch.Tensor, params: list, counters: list, seeds: list, generated: list):
        """As `sample`, without waiting: returns a PendingSample.  At most two may be outstanding (the result
        buffers alternate), and one's `tokens_device` is overwritten by the launch after it."""
        rows = logits.shape[0]
        if rows == 0:
            return PendingSample(0, None, None, None, None)
        if self._side is None:
            self._staging = load_family("staging")
            self._side = torch.cuda.Stream(self.device)
            self._side_raw = c_void_p(self._side.cuda_stream)
            self._queued = new_event(self._staging)
            self._done = [new_event(self._staging), new_event(self._staging)]
        lib = self._staging
        if self._read is not None:
            # the copy out of the previous results is done (it has long been) before the next launch overwrites them
            ops._check(lib.wllm_stream_wait(ops._stream(), self._read), "ordering the sampler behind its last copy")
        tokens = self.launch(logits, params, counters, seeds, generated)
        self._turn ^= 1
        host = self._out_hosts[self._turn]
        if host is None or host[0].numel() < 2 * rows + 1:
            pinned = torch.empty(max(2 * rows + 1, 1024), dtype=torch.int32).pin_memory()
            host = self._out_hosts[self._turn] = (pinned, pinned.numpy())
        done = self._done[self._turn]
        # the copy to the host runs on a stream of its own and leaves the step's stream free for the next step's first kernels
        ops._check(lib.wllm_stage_fetch(c_void_p(host[0].data_ptr()), c_void_p(self._out.data_ptr()), c_longlong(8 * rows),
                                        c_void_p(ops._status_word(self.device).data_ptr()), c_longlong(4),
                                        ops._stream(), self._side_raw, self._queued, done), "copy of the sampled ids")
        self._read = done
        self.d2h_bytes = 8 * rows + 4
        return PendingSample(rows, tokens, host[1], done, lib, self)

    def _scratch_for(self, rows: int, lib) -> c_void_p:
        need = int(lib.wllm_sample_scratch_row_bytes()) * max(rows, 64)
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.zeros(need, dtype=torch.uint8, device=self.device)
        return c_void_p(self._scratch.data_ptr())

    def _launch_greedy(self, logits: torch.Tensor) -> torch.Tensor:
        """All rows greedy and unpenalised: no options to send, and the first pass alone."""
        rows, V = logits.shape
        if self._out is None or self._out.numel() < 2 * rows:
            self._out = torch.empty(max(2 * rows, 1024), dtype=torch.int32, device=self.device)
        lib = load_family("sampling")
        ops._check(lib.wllm_sample_greedy(c_void_p(logits.data_ptr()), logits.stride(0), rows, V, self._scratch_for(rows, lib),
                                          c_void_p(self._out.data_ptr()), c_void_p(self._out.data_ptr() + 4 * rows),
                                          ops._stream()), "sample_greedy")
        ops.launches += 1
        self.h2d_bytes = 0
        return self._out[:rows]

    def launch(self, logits: torch.Tensor, params: list, counters: list, seeds: list, generated: list):
        """Enqueue the sampling of all rows; tokens [rows] int32 stay on the device (returned view)."""
        rows, V = logits.shape
        if logits.dtype != torch.float32 or logits.stride(1) != 1:
            raise ops.KernelError("sampling needs float32 logits with unit stride along the vocabulary")
        if all(p.temperature == 0.0 and p.repetition_penalty == 1.0 for p in params):
            return self._launch_greedy(logits)
        host, filters = pack_options(params, counters, seeds, generated)
        if self._dev is None or self._dev.numel() < host.shape[0]:
            self._dev = torch.empty(max(host.shape[0], 8192), dtype=torch.int32, device=self.device)
        self._ring.send(host, self._dev)
        self.h2d_bytes = host.shape[0] * 4
        return self.launch_packed(logits, filters)

    def launch_packed(self, logits: torch.Tensor, filters: int) -> torch.Tensor:
        """The kernels alone, on the options that the last `launch` left on the device."""
        rows, V = logits.shape
        if self._out is None or self._out.numel() < 2 * rows:
            self._out = torch.empty(max(2 * rows, 1024), dtype=torch.int32, device=self.device)
        lib = load_family("sampling")
        scratch = self._scratch_for(rows, lib)
        base = self._dev.data_ptr()

        def at(i):
            return c_void_p(base + 4 * i)
        launched = c_int(0)
        ops._check(lib.wllm_sample(c_void_p(logits.data_ptr()), logits.stride(0), rows, V, at(0), at(rows), at(2 * rows),
                                   at(3 * rows), at(4 * rows), at(5 * rows), at(6 * rows), at(7 * rows), at(8 * rows),
                                   at(9 * rows + 1), scratch, filters,
                                   c_void_p(self._out.data_ptr()), c_void_p(self._out.data_ptr() + 4 * rows),
                                   byref(launched), ops._stream()), "sample")
        ops.launches += launched.value
        return self._out[:rows]


def pack_options(params: list, counters: list, seeds: list, generated: list):
    """One int32 array with, row by row in this order: temperature, top-k, top-p, min-p, penalty, the seed's
    lower and upper half, the counter, the offsets of each row's generated ids, and those ids; and which
    selection passes some row needs (bit 0: any filter, bit 1: top-k or top-p)."""
    rows = len(params)
    gen_lists = [sorted(g) if p.repetition_penalty != 1.0 else [] for p, g in zip(params, generated)]
    offsets = np.zeros(rows + 1, dtype=np.int32)
    offsets[1:] = np.cumsum([len(g) for g in gen_lists])
    n_gen = int(offsets[-1])
    host = np.zeros(8 * rows + (rows + 1) + n_gen, dtype=np.int32)
    f = host.view(np.float32)
    f[0:rows] = [p.temperature for p in params]
    host[rows:2 * rows] = [p.top_k for p in params]
    f[2 * rows:3 * rows] = [p.top_p for p in params]
    f[3 * rows:4 * rows] = [p.min_p for p in params]
    f[4 * rows:5 * rows] = [p.repetition_penalty for p in params]
    s = np.asarray([x & 0xFFFFFFFFFFFFFFFF for x in seeds], dtype=np.uint64)
    host[5 * rows:6 * rows] = (s & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.int32)
    host[6 * rows:7 * rows] = (s >> np.uint64(32)).astype(np.uint32).view(np.int32)
    host[7 * rows:8 * rows] = counters
    host[8 * rows:9 * rows + 1] = offsets
    if n_gen:
        host[9 * rows + 1:] = np.concatenate([np.asarray(g, dtype=np.int32) for g in gen_lists if g])
    sampled = [p for p in params if p.temperature != 0.0]
    filters = (1 if any(p.top_k > 0 or p.top_p < 1.0 or p.min_p > 0.0 for p in sampled) else 0) | \
              (2 if any(p.top_k > 0 or p.top_p < 1.0 for p in sampled) else 0)
    return host, filters
