"""Continuous batching above the step function.

Every step is ONE batch for `ModelRunner.step`: each decoding request brings its newest
token, each prefilling request the next portion of its prompt, and newly admitted
requests their first portion; whoever's known tokens are all in the cache after the
step gets one sampled token.  So a request advances by at most one token per step, as
in the reference (src/wllm/engine/scheduler.py:454-498), which however runs one forward
per prefilling request and one more for the decoding batch.

Policy, with the reference's rule beside it:
  admission   first come first served, the head of the queue blocks those behind it
              (scheduler.py:192-205).  'worst_case' (default): admit when the pages for
              prompt + max_tokens fit into the free pages minus what live requests may
              still claim (scheduler.py:181-199, but counted from pages actually held).
              'optimistic': admit when the prompt's pages are free now.
  budget      `chunked_prefill_tokens` bounds the prompt tokens of one step; requests
              already prefilling come first, in order of admission, then new ones, each
              taking min(budget left, tokens left) (scheduler.py:215-257).  Decoded
              tokens ride along uncounted.  None: whole prompts.
  rows        `row_quantum` (no counterpart in the reference; 0 = off): the matrix products of a
              step of many rows work on tiles of that many rows (256 for the bfloat16 products
              on pairs of CTAs), so 2,048 prompt tokens beside 52 decoded ones cost nine tiles
              of rows where 1,996 cost eight.  When the budget and the decoded tokens together
              pass a multiple of the quantum, the budget of that step is cut back to the
              multiple if that gives more prompt tokens a tile; the tokens cut come next step.
  pages out   the step reserves all its pages first; on OutOfPages the youngest live
              request is preempted: its pages go back, it returns to the FRONT of the
              queue and is later run again from its prompt plus the tokens it has
              generated, which it keeps (the reference discards them, scheduler.py:293-305).
              A seeded request continues exactly as it would have.  A request that could
              not run even alone is refused when it is added, so the loop cannot spin.
  finishing   end-of-sequence id, stop ids, max_tokens or the model's length; pages are
              given back in the same step (scheduler.py:492-495).
  pipelining  `async_scheduling` (no counterpart in the reference): step k+1 is planned and
              launched before the host has read the tokens of step k.  Its decode entries
              take their token from the device, where the sampler left it; the host reads
              step k's tokens while step k+1 runs, so `step()` returns the tokens of the
              step before.  A request that turns out to have stopped at step k has then
              already run in step k+1: that token is dropped, its pages are given back
              (the device runs in stream order, so whoever gets them writes later).
              max_tokens and the model's length are known by count and waste nothing.
              A repetition penalty needs every earlier token on the host, and a shortage
              of pages is settled with nothing in flight: both read the tokens first.
"""
from __future__ import annotations

import random

from ..cache import OutOfPages
from .request import Request, RequestStatus
from .runner import StepEntry


class Scheduler:
    def __init__(self, runner, sampler, chunked_prefill_tokens: int | None = None, max_num_seqs: int = 256,
                 max_model_len: int | None = None, admission: str = "worst_case", seed: int = 0,
                 async_scheduling: bool = False, row_quantum: int = 0):
        if admission not in ("worst_case", "optimistic"):
            raise ValueError("admission must be 'worst_case' or 'optimistic'")
        self.runner, self.sampler, self.cache = runner, sampler, runner.cache
        self.budget = chunked_prefill_tokens
        self.row_quantum = int(row_quantum)
        self.max_num_seqs = min(max_num_seqs, self.cache.slots.num_slots)
        self.max_model_len = max_model_len or runner.model.plan.max_positions
        self.admission = admission
        self.waiting: list = []
        self.live: list = []          # admitted requests in order of admission
        self._rng = random.Random(seed)
        self.async_scheduling = async_scheduling
        self._inflight = None         # (PendingSample, [(request, keep)]) of the step whose tokens are unread
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0, "finished": 0,
                      "dropped_tokens": 0}

    # -- requests ------------------------------------------------------------------------
    def _pages(self, tokens: int) -> int:
        return -(-tokens // self.cache.page_size)

    def add_request(self, request: Request) -> None:
        n = len(request.prompt_token_ids)
        if n == 0:
            raise ValueError(f"request {request.request_id!r}: empty prompt")
        if n >= self.max_model_len:
            raise ValueError(f"request {request.request_id!r}: prompt of {n} tokens leaves no room under the "
                             f"model length {self.max_model_len}")
        vocab = self.runner.model.plan.vocab_size
        bad = [t for t in request.prompt_token_ids if not 0 <= t < vocab]
        if bad:
            raise ValueError(f"request {request.request_id!r}: token id {bad[0]} outside the vocabulary of {vocab}")
        worst = min(request.worst_case_tokens, self.max_model_len)
        pool = min(g.pool.num_pages for g in self.cache.groups) if self.cache.groups else 1 << 30
        if self._pages(worst) > pool:
            raise ValueError(f"request {request.request_id!r}: {worst} tokens need {self._pages(worst)} pages, "
                             f"the cache has {pool}; it could never finish")
        request.status = RequestStatus.WAITING
        request.seed = request.sampling.seed if request.sampling.seed is not None else self._rng.getrandbits(63)
        self.waiting.append(request)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.live or self._inflight)

    def cancel(self, request_id) -> bool:
        """Stop a request wherever it is and give back what it holds (scheduler.py:158-176)."""
        for r in self.live:
            if r.request_id == request_id:
                self._release(r)
                self.live.remove(r)
                r.status, r.finish_reason = RequestStatus.FINISHED, "cancelled"
                return True
        for r in self.waiting:
            if r.request_id == request_id:
                self.waiting.remove(r)
                r.status, r.finish_reason = RequestStatus.FINISHED, "cancelled"
                return True
        return False

    def _release(self, r: Request) -> None:
        if r.cache is not None:
            self.cache.close(r.cache)
            r.cache = None
        r.num_computed = 0
        r.inflight = 0

    # -- admission -------------------------------------------------------------------------
    def _pledged(self) -> int:
        """Pages that live requests may still claim before they finish."""
        total = 0
        for r in self.live:
            worst = self._pages(min(r.worst_case_tokens, self.max_model_len))
            held = max((len(t) for t in r.cache.tables), default=0)
            total += max(0, worst - held)
        return total

    def _may_admit(self, r: Request, taken_now: int) -> bool:
        if len(self.live) >= self.max_num_seqs:
            return False
        free = min(self.cache.free_pages(), default=1 << 30)
        if self.admission == "worst_case":   # the pledge covers the pages this step is about to take
            return self._pages(min(r.worst_case_tokens, self.max_model_len)) <= free - self._pledged()
        return self._pages(r.num_tokens) <= free - taken_now

    def _preempt_youngest(self) -> Request:
        victim = self.live.pop()
        self._release(victim)
        victim.status = RequestStatus.WAITING
        victim.preemptions += 1
        self.waiting.insert(0, victim)
        self.stats["preemptions"] += 1
        return victim

    # -- one step ----------------------------------------------------------------------------
    def _last_in_flight(self, r: Request) -> bool:
        """With pipelining: the token in flight is the request's last, so it brings nothing to this step."""
        return bool(r.inflight) and (len(r.output_token_ids) + 1 >= r.sampling.max_tokens
                                     or r.num_tokens + 1 >= self.max_model_len)

    def _step_budget(self) -> int:
        """The prompt tokens this step may take: the budget, cut back to where the step's rows (decoded tokens ride
        along) are a multiple of `row_quantum` when that gives more prompt tokens per tile of rows."""
        if self.budget is None:
            return 1 << 60
        q, budget = self.row_quantum, self.budget
        if q <= 0:
            return budget
        riding = sum(1 for r in self.live if r.status == RequestStatus.RUNNING and not self._last_in_flight(r))
        rows = budget + riding
        cut = rows // q * q - riding
        if rows % q == 0 or rows < q or cut < 1:
            return budget
        return cut if cut * -(-rows // q) > budget * (rows // q) else budget      # cut / tiles' > budget / tiles

    def _plan(self):
        """(request, first token index, count) for this step; admits from the queue."""
        budget = self._step_budget()
        plan, taken = [], 0
        for r in self.live:
            left = r.num_tokens + r.inflight - r.num_computed
            if r.status == RequestStatus.RUNNING:
                if self._last_in_flight(r):
                    continue                               # the token in flight is its last
                plan.append((r, r.num_computed, left))     # its newest token (one), outside the budget
                continue
            if budget <= 0:
                continue
            c = min(budget, left)
            budget -= c
            plan.append((r, r.num_computed, c))
        for r, _, c in plan:
            taken += max(self.cache.pages_needed([(r.cache, c)]), default=0)     # of the group that needs most
        while self.waiting and budget > 0:
            r = self.waiting[0]
            if not self._may_admit(r, taken):
                break                                       # the head of the queue blocks the rest
            self.waiting.pop(0)
            r.cache = self.cache.open(r.request_id)
            r.num_computed = 0
            r.status = RequestStatus.PREFILLING
            self.live.append(r)
            c = min(budget, r.num_tokens)
            budget -= c
            plan.append((r, 0, c))
            taken += self._pages(c)
        return plan

    def _resolve(self) -> list:
        """Read the tokens of the step in flight and give them to their requests; finish and free."""
        if self._inflight is None:
            return []
        pending, rows = self._inflight
        self._inflight = None
        tokens, logprobs = pending.get()
        got = []
        for (r, keep), t, lp in zip(rows, tokens, logprobs):
            if not keep or r.finished or r.inflight == 0:
                self.stats["dropped_tokens"] += 1
                continue
            r.inflight = 0
            r.append_token(int(t), float(lp), self.max_model_len)
            got.append(r)
        self._finish()
        return got

    def _finish(self) -> None:
        for r in [r for r in self.live if r.finished]:
            self._release(r)
            self.live.remove(r)
            self.stats["finished"] += 1

    def _entry(self, r: Request, start: int, c: int) -> StepEntry:
        want = [c - 1] if start + c == r.num_tokens + r.inflight else []
        if r.inflight:
            return StepEntry(r.cache, [0], want, device_row=r.inflight_row)
        return StepEntry(r.cache, r.tokens(start, start + c), want)

    def step(self) -> list:
        """One batch.  Returns the requests that got a token on the host in this call: those sampled in this
        step, or with `async_scheduling` those of the step before."""
        got = []
        if self._inflight and any(r.sampling.repetition_penalty != 1.0 for r in self.live):
            got += self._resolve()
        plan = self._plan()
        while True:
            if not plan:
                if self._inflight:
                    return self._once(got + self._resolve())
                if self.waiting and not self.live:
                    raise RuntimeError(f"request {self.waiting[0].request_id!r} cannot be admitted into an empty engine")
                return got
            entries = [self._entry(r, start, c) for r, start, c in plan]
            try:
                if self._inflight:
                    logits = self.runner.step(entries, device_tokens=self._inflight[0].tokens_device)
                else:
                    logits = self.runner.step(entries)
                break
            except OutOfPages:
                if self._inflight:            # settle it with every token on the host
                    got += self._resolve()
                    plan = self._plan()
                    continue
                if len(self.live) <= 1:
                    raise
                victim = self._preempt_youngest()
                plan = [p for p in plan if p[0] is not victim]
        self.stats["steps"] += 1
        sampled = []
        for r, start, c in plan:
            if r.status == RequestStatus.RUNNING:
                self.stats["decode_tokens"] += c
            else:
                self.stats["prefill_tokens"] += c
            r.num_computed = start + c
            if r.num_computed == r.num_tokens + r.inflight:
                sampled.append(r)
        args = ([r.sampling for r in sampled], [len(r.output_token_ids) + r.inflight for r in sampled],
                [r.seed for r in sampled], [r.seen for r in sampled])
        if not self.async_scheduling:
            if sampled:
                tokens, logprobs = self.sampler.sample(logits, *args)
                for r, t, lp in zip(sampled, tokens, logprobs):
                    r.status = RequestStatus.RUNNING
                    r.append_token(int(t), float(lp), self.max_model_len)
            self._finish()
            return sampled
        pending = self.sampler.sample_pending(logits, *args) if sampled else None
        got += self._resolve()                 # the step before, while this one runs
        if pending is not None:
            rows = []
            for row, r in enumerate(sampled):
                keep = not r.finished          # it may just have turned out to have stopped a step ago
                if keep:
                    r.status, r.inflight, r.inflight_row = RequestStatus.RUNNING, 1, row
                rows.append((r, keep))
            self._inflight = (pending, rows)
            if any(r.sampling.repetition_penalty != 1.0 for r in sampled):
                got += self._resolve()
        return self._once(got)

    @staticmethod
    def _once(requests: list) -> list:
        seen, out = set(), []
        for r in requests:
            if id(r) not in seen:
                seen.add(id(r))
                out.append(r)
        return out

    def run_to_completion(self, max_steps: int | None = None) -> list:
        """Step until nothing is left (scheduler.py:500-506); returns finished requests in finishing order."""
        done, steps = [], 0
        while self.has_unfinished():
            for r in self.step():
                if r.finished:
                    done.append(r)
            steps += 1
            if max_steps is not None and steps >= max_steps:
                break
        return done
