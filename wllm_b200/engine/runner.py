"""The step function: one batch of (request, its next tokens) through the model.

`ModelRunner.step(entries)` takes portions of prompts beside single decoded tokens,
cut anywhere, runs exactly the tokens it is given against the cache that earlier
steps left, and returns the 32-bit logits at the wanted places (device tensor
[wanted, vocab], in the order of the entries and of their `want`).  It reserves the
pages for the whole batch first (all or nothing: `OutOfPages` leaves everything as
it was), builds the batch's index arrays on the host, sends them in one copy, runs
the model, and commits the new tokens.

The reference has three separate forwards instead (whole prompt, one portion, batch
of decoded tokens: src/wllm/models/llama.py:448-560) and never mixes them in one pass.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from ..cache import CacheManager, RequestCache
from ..kernels import ops
from .model import ComposedModel
from .staging import PinnedRing


@dataclass
class StepEntry:
    cache: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()
    # The entry's single token is not known on the host yet: it is row `device_row` of the `device_tokens`
    # given to `step` (what the sampler left on the device); `tokens` then holds one placeholder.
    device_row: int | None = None


class StepContext:
    """The batch as the parts see it: index arrays on the device (and the same on the host, for launch decisions),
    the cache, scratch buffers, and a few facts about the batch's shape (how many requests bring one token and how
    many several, the longest portion, the longest context).  It chooses no kernel: that is the parts' business."""

    def __init__(self, runner: "ModelRunner"):
        self.runner = runner
        self.cache = runner.cache
        self.n_tokens = self.n_requests = 0
        self.token_ids = self.positions = self.token_req = self.want_rows = None
        self.req_q_start = self.req_q_len = self.req_ctx_len = self.req_slot = None
        self.group_slots: list = []
        self.group_tables: list = []
        self.host = None   # the same arrays on the host, for launch decisions
        self.num_single = self.num_multi = 0     # requests with one token / with several
        self.memo: dict = {}                     # what a part worked out for this step and wants again in the next layer
        self.max_q_len = self.max_ctx = 0        # bounds that size the attention grids

    def buffer(self, name: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        return self.runner.workspace(name, shape, dtype)

    def state(self, name: str) -> torch.Tensor:
        return self.cache.slots.tensors[name]


class ModelRunner:
    def __init__(self, model: ComposedModel, cache: CacheManager, device):
        if not model.loaded:
            raise RuntimeError("the model's weights are not loaded")
        self.model, self.cache, self.device = model, cache, torch.device(device)
        self._arena: dict = {}
        self._views: dict = {}         # (name, shape, dtype) -> the view handed out before
        self._ring = PinnedRing(self.device)
        self._meta = None
        self.steps = 0
        self.tokens_run = 0
        self.h2d_bytes = 0
        self._tables: dict = {}        # cached int32 copies of block tables
        self._graphs_on = False
        self._graphs: dict = {}        # (requests, table width) -> captured decode step
        self.graph_launches = 0        # kernel launches replayed from graphs so far

    def workspace(self, name: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        """A scratch tensor of that shape at the front of the arena's buffer of that name and type (the same memory
        for every shape asked under the name; the buffer grows when a larger one is asked for)."""
        view = self._views.get((name, shape, dtype))
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= s
        key = (name, dtype)
        buf = self._arena.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._arena[key] = buf
            for k in [k for k in self._views if k[0] == name and k[2] == dtype]:
                del self._views[k]                  # views of the buffer that this one replaces
        if len(self._views) > 4096:
            self._views.clear()
        view = self._views[(name, shape, dtype)] = buf[:n].view(shape)
        return view

    # -- batch building --------------------------------------------------------------
    def _host_arrays(self, entries: list, table_width: int | None, pad_requests: int | None):
        """The step's index arrays in one int32 host array: (array, {name: (offset, length)}, names in order,
        (tokens, requests, table width), patches)."""
        cache, ps = self.cache, self.cache.page_size
        G, real = len(cache.groups), len(entries)
        lens = [len(e.tokens) for e in entries]
        P = table_width or max(1, max(len(t) for e in entries for t in e.cache.tables) if G else 1)
        if pad_requests is not None:
            assert sum(lens) == real and pad_requests >= real
            R = N = M = pad_requests
        else:
            R, N, M = real, sum(lens), sum(len(e.want) for e in entries)

        def pad(n):
            return (n + 3) & ~3
        sizes = [("token_ids", N), ("positions", N), ("token_req", N)] + [(f"slots{g}", N) for g in range(G)] + \
                [("req_q_start", R), ("req_q_len", R), ("req_ctx_len", R), ("req_slot", R), ("want_rows", M)] + \
                [(f"table{g}", R * P) for g in range(G)] + [("patch_dst", R), ("patch_src", R)]
        offsets, total = {}, 0
        for name, n in sizes:
            offsets[name] = (total, n)
            total += pad(n)
        host = np.zeros(total, dtype=np.int32)

        def view(name):
            o, n = offsets[name]
            return host[o:o + n]
        start = 0
        wants = []
        if N == R:
            # every request brings one token (a decode step): whole columns at once, tables from cached copies
            bases = [e.cache.num_tokens for e in entries]
            view("token_ids")[:real] = [e.tokens[0] for e in entries]
            view("positions")[:real] = bases
            ar = np.arange(R, dtype=np.int32)
            view("token_req")[:] = ar
            view("req_q_start")[:] = ar
            view("req_q_len")[:real] = 1
            view("req_ctx_len")[:real] = np.asarray(bases, dtype=np.int32) + 1
            view("req_slot")[:real] = [e.cache.slot for e in entries]
            for g in range(G):
                view(f"slots{g}")[real:] = -1
                view(f"slots{g}")[:real] = [e.cache.tables[g][b // ps] * ps + b % ps for e, b in zip(entries, bases)]
                rows2d = view(f"table{g}").reshape(R, P)
                for r, e in enumerate(entries):
                    t = self._table_copy(e.cache, g)
                    rows2d[r, :t.shape[0]] = t
            if pad_requests is not None:
                wants.extend(range(R))
            else:
                for r, e in enumerate(entries):
                    wants.extend(r + w for w in e.want)
            entries_loop = ()
        else:
            entries_loop = enumerate(entries)
        for r, e in entries_loop:
            n, base = lens[r], e.cache.num_tokens
            view("token_ids")[start:start + n] = e.tokens
            view("positions")[start:start + n] = np.arange(base, base + n, dtype=np.int32)
            view("token_req")[start:start + n] = r
            for g in range(G):
                table = np.asarray(e.cache.tables[g], dtype=np.int64)
                pos = np.arange(base, base + n, dtype=np.int64)
                view(f"slots{g}")[start:start + n] = table[pos // ps] * ps + pos % ps
                view(f"table{g}").reshape(R, P)[r, :len(table)] = table
            view("req_q_start")[r], view("req_q_len")[r] = start, n
            view("req_ctx_len")[r], view("req_slot")[r] = base + n, e.cache.slot
            wants.extend(start + w for w in e.want)
            start += n
        view("want_rows")[:] = wants
        patches = [(r, e.device_row) for r, e in enumerate(entries) if e.device_row is not None]
        if patches:
            starts = np.cumsum([0] + lens[:-1])
            view("patch_dst")[:len(patches)] = [starts[r] for r, _ in patches]
            view("patch_src")[:len(patches)] = [row for _, row in patches]

        return host, offsets, [k for k, _ in sizes], (N, R, P), patches

    def _send(self, host, offsets, patches, device_tokens) -> None:
        """The host array to the device's index buffer; tokens that lie on the device are put in their places."""
        total = host.shape[0]
        if self._meta is None or self._meta.numel() < total:
            cap = max(total, 4096, 2 * (self._meta.numel() if self._meta is not None else 0))
            self._graphs.clear()      # captured steps point into the old index buffer
            self._meta = torch.empty(cap, dtype=torch.int32, device=self.device)
        self._ring.send(host, self._meta)
        self.h2d_bytes = total * 4
        if patches:
            def dev(name, n):
                o = offsets[name][0]
                return self._meta[o:o + n]
            ops.patch_tokens(dev("token_ids", offsets["token_ids"][1]), dev("patch_dst", len(patches)), device_tokens,
                             dev("patch_src", len(patches)))

    def _build(self, entries: list, table_width: int | None = None, device_tokens=None,
               pad_requests: int | None = None) -> StepContext:
        """`pad_requests` (a decode step under a captured graph): the arrays are laid out for that many requests;
        the ones behind the real entries bring no token (q_len 0, no cache slot), so every kernel passes them
        by, and the logits of all rows are wanted (the caller keeps the real ones)."""
        host, offsets, names, (N, R, P), patches = self._host_arrays(entries, table_width, pad_requests)
        self._send(host, offsets, patches, device_tokens)
        ps, real = self.cache.page_size, len(entries)
        lens = [len(e.tokens) for e in entries]
        G = len(self.cache.groups)

        def view(name):
            o, n = offsets[name]
            return host[o:o + n]
        ctx = StepContext(self)
        ctx.n_tokens, ctx.n_requests, ctx.host = N, R, {k: view(k) for k in names}
        ctx.host["max_pages"] = P
        ctx.num_single = sum(1 for n in lens if n == 1)
        ctx.num_multi = real - ctx.num_single
        ctx.max_q_len = max(lens)
        # under a captured graph the bound must not depend on the batch's contents: the table's reach
        ctx.max_ctx = table_width * ps if table_width else max(e.cache.num_tokens + n for e, n in zip(entries, lens))

        def dev(name):
            o, n = offsets[name]
            return self._meta[o:o + n]
        ctx.token_ids, ctx.positions, ctx.token_req = dev("token_ids"), dev("positions"), dev("token_req")
        ctx.req_q_start, ctx.req_q_len = dev("req_q_start"), dev("req_q_len")
        ctx.req_ctx_len, ctx.req_slot, ctx.want_rows = dev("req_ctx_len"), dev("req_slot"), dev("want_rows")
        ctx.group_slots = [dev(f"slots{g}") for g in range(G)]
        ctx.group_tables = [dev(f"table{g}").view(R, P) for g in range(G)]
        return ctx

    def _table_copy(self, rc, group: int) -> np.ndarray:
        """A request's block table of one group as an int32 array, rebuilt only when the table changed."""
        key = (id(rc), group)
        hit = self._tables.get(key)
        if hit is None or hit[0] != rc.version or hit[2] is not rc:
            if len(self._tables) > 4096:
                self._tables.clear()
            hit = (rc.version, np.asarray(rc.tables[group], dtype=np.int32), rc)
            self._tables[key] = hit
        return hit[1]

    def _validate(self, entries: list) -> None:
        vocab, limit = self.model.plan.vocab_size, self.model.plan.max_positions
        seen = set()
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.cache.request_id!r}: an entry needs at least one token")
            if id(e.cache) in seen:
                raise ValueError(f"request {e.cache.request_id!r} appears twice in one step")
            seen.add(id(e.cache))
            if e.cache.closed:
                raise ValueError(f"request {e.cache.request_id!r} is closed")
            if e.cache.num_tokens + n > limit:
                raise ValueError(f"request {e.cache.request_id!r}: {e.cache.num_tokens + n} tokens exceed the "
                                 f"model's {limit} positions")
            if e.device_row is not None and n != 1:
                raise ValueError(f"request {e.cache.request_id!r}: a token taken from the device stands alone")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= vocab:
                raise ValueError(f"request {e.cache.request_id!r}: token id {lo if lo < 0 else hi} outside the "
                                 f"vocabulary of {vocab}")
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.cache.request_id!r}: wanted place {w} outside its {n} tokens")

    # -- captured decode steps -------------------------------------------------------------
    def enable_graphs(self) -> None:
        """Replay a captured CUDA graph for steps in which every request brings one token and
        wants its logits (a decode step), if every part of the model is `graph_safe` and none keeps
        per-request state; other models step eagerly.  One graph per (number of requests, table width);
        the index arrays live at fixed device addresses and are rewritten before each replay.
        The reference captures its decode step in batch-size buckets the same way
        (src/wllm/engine/cuda_graph_decoder.py:34-178)."""
        self._graphs_on = True

    def _graphable(self, entries: list) -> bool:
        return self._graphs_on and self.model.graph_safe and \
            all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)

    def _forward_graph(self, entries: list, device_tokens=None) -> torch.Tensor:
        widest = max(1, max(len(t) for e in entries for t in e.cache.tables))
        width = 8
        while width < widest:
            width *= 2
        bucket = 1                      # 1, 2, 3, 4, 6, 8, 12, 16, 24, 32, ...: a capture serves every count up to its size
        while bucket < len(entries):
            bucket = bucket * 3 // 2 if bucket & (bucket - 1) == 0 and bucket > 1 else (bucket * 4 // 3 if bucket > 2 else bucket + 1)
        key = (bucket, width)
        rec = self._graphs.get(key)
        if rec is not None:
            # a replay reads the index buffer at the addresses of its capture: the arrays go there, nothing else is built
            host, offsets, _, _, patches = self._host_arrays(entries, width, bucket)
            self._send(host, offsets, patches, device_tokens)
            rec = self._graphs.get(key)         # the send may have had to grow the buffer, which drops the captures
        if rec is None:
            ctx = self._build(entries, table_width=width, device_tokens=device_tokens, pad_requests=bucket)
            arena, saved, saved_views = {}, self._arena, self._views
            self._arena, self._views = arena, {}     # the capture's buffers are its own: eager steps do not write them
            try:
                self.model.forward(ctx)                  # loads kernels and library handles outside the capture
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                before = ops.launches
                with torch.cuda.graph(graph):
                    logits = self.model.forward(ctx)
                rec = {"graph": graph, "logits": logits, "arena": arena, "launches": ops.launches - before,
                       "meta": self._meta}
                ops.launches = before
            finally:
                self._arena, self._views = saved, saved_views
            self._graphs[key] = rec
        rec["graph"].replay()
        self.graph_launches += rec["launches"]
        return rec["logits"][:len(entries)]

    # -- the step ----------------------------------------------------------------------
    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """`device_tokens`: int32 tokens on the device, read by the entries that name a `device_row`."""
        entries = list(entries)
        if not entries:
            return torch.empty((0, self.model.plan.vocab_size), dtype=torch.float32, device=self.device)
        self._validate(entries)
        if device_tokens is None and any(e.device_row is not None for e in entries):
            raise ValueError("an entry names a device row, but no device tokens were given")
        self.cache.reserve([(e.cache, len(e.tokens)) for e in entries])   # all or nothing
        try:
            if self._graphable(entries):
                logits = self._forward_graph(entries, device_tokens)
                ctx = None
            else:
                ctx = self._build(entries, device_tokens=device_tokens)
                logits = self.model.forward(ctx)
        except BaseException:
            for e in entries:          # a failed step holds no pages beyond its committed tokens
                self.cache.cancel_reservation(e.cache)
            raise
        for e in entries:
            self.cache.commit(e.cache, len(e.tokens))
        self.steps += 1
        self.tokens_run += sum(len(e.tokens) for e in entries)
        return logits
