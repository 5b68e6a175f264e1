"""The scheduler's decisions on the host, with a stand-in for the step function: who is
admitted, how prompts are cut under the budget, one token per request and step, finishing,
and what happens when pages run out."""
import pytest
import torch

from wllm_b200.cache import CacheGroupSpec, CacheManager
from wllm_b200.engine.request import Request, RequestStatus
from wllm_b200.engine.scheduler import Scheduler
from wllm_b200.sampling import SamplingParams

VOCAB = 50


class FakePlan:
    vocab_size, max_positions = VOCAB, 64


class FakeModel:
    plan = FakePlan()


class FakeRunner:
    """Reserves and commits like the real step function and returns logits that make the next
    token a fixed function of (last token, position), so outputs do not depend on the cut."""

    def __init__(self, pages, page_size=4, max_requests=8):
        self.cache = CacheManager([CacheGroupSpec("all", 1, 1, 8)], page_size, pages, max_requests)
        self.model = FakeModel()
        self.batches = []
        self.from_device = []      # per step: entries whose token came from the step before, unread by the host

    def step(self, entries, device_tokens=None):
        self.cache.reserve([(e.cache, len(e.tokens)) for e in entries])
        rows = []
        for e in entries:
            tokens = list(e.tokens) if e.device_row is None else [device_tokens[e.device_row]]
            for w in e.want:
                pos = e.cache.num_tokens + w
                row = torch.zeros(VOCAB)
                row[(tokens[w] * 7 + pos * 3 + 1) % VOCAB] = 1.0
                rows.append(row)
        self.batches.append([(e.cache.request_id, len(e.tokens), list(e.want)) for e in entries])
        self.from_device.append(sum(e.device_row is not None for e in entries))
        for e in entries:
            self.cache.commit(e.cache, len(e.tokens))
        self.cache.check()
        return torch.stack(rows) if rows else torch.zeros(0, VOCAB)


class Pending:
    def __init__(self, tokens):
        self.tokens_device, self.reads = tokens, 0

    def get(self):
        self.reads += 1
        return self.tokens_device, [0.0] * len(self.tokens_device)


class ArgmaxSampler:
    def __init__(self):
        self.seen_at_launch = []

    def sample(self, logits, params, counters, seeds, generated):
        return logits.argmax(-1).tolist(), [0.0] * logits.shape[0]

    def sample_pending(self, logits, params, counters, seeds, generated):
        self.seen_at_launch.append((list(counters), [set(g) for g in generated]))
        return Pending(logits.argmax(-1).tolist())


def expected_output(prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        t = (toks[-1] * 7 + (len(toks) - 1) * 3 + 1) % VOCAB
        out.append(t)
        toks.append(t)
    return out


def make(pages=16, budget=None, **kw):
    runner = FakeRunner(pages)
    return Scheduler(runner, ArgmaxSampler(), chunked_prefill_tokens=budget, **kw), runner


def req(i, n, max_tokens=4, **kw):
    return Request(i, [(i * 5 + j) % VOCAB for j in range(n)], SamplingParams(max_tokens=max_tokens, **kw))


def test_whole_prompts_then_one_token_per_step():
    s, runner = make()
    a, b = req(0, 5, 3), req(1, 9, 3)
    s.add_request(a); s.add_request(b)
    got = s.step()
    assert runner.batches[0] == [(0, 5, [4]), (1, 9, [8])] and got == [a, b]
    assert [len(r.output_token_ids) for r in (a, b)] == [1, 1] and a.status == RequestStatus.RUNNING
    s.step()
    assert runner.batches[1] == [(0, 1, [0]), (1, 1, [0])]
    s.run_to_completion()
    assert a.output_token_ids == expected_output(a.prompt_token_ids, 3) and a.finish_reason == "length"
    assert b.output_token_ids == expected_output(b.prompt_token_ids, 3)
    assert runner.cache.free_pages() == [16] and not s.has_unfinished()


def test_budget_cuts_prompts_and_decodes_ride_along():
    s, runner = make(pages=32, budget=6)
    a, b, c = req(0, 4, 5), req(1, 11, 2), req(2, 3, 2)
    for r in (a, b, c):
        s.add_request(r)
    s.step()   # a whole (4), b gets the remaining 2; c waits for budget
    assert runner.batches[0] == [(0, 4, [3]), (1, 2, [])]
    assert a.status == RequestStatus.RUNNING and b.status == RequestStatus.PREFILLING and c.status == RequestStatus.WAITING
    s.step()   # a decodes outside the budget; b continues with 6
    assert runner.batches[1] == [(0, 1, [0]), (1, 6, [])]
    s.step()   # b's last 3 complete it, c is admitted with what is left of the budget
    assert runner.batches[2] == [(0, 1, [0]), (1, 3, [2]), (2, 3, [2])]
    assert len(b.output_token_ids) == 1 and len(c.output_token_ids) == 1 and len(a.output_token_ids) == 3
    s.run_to_completion()
    for r in (a, b, c):
        assert r.output_token_ids == expected_output(r.prompt_token_ids, r.sampling.max_tokens)


def test_the_budget_is_cut_back_to_whole_tiles_of_rows_when_that_gives_more_prompt_tokens_a_tile():
    """row_quantum 8, budget 16.  Alone, a prompt takes 16 tokens a step (two tiles of rows).  With 3 requests
    decoding beside it, 16 + 3 rows would be three tiles for 16 prompt tokens; 13 + 3 are two tiles for 13: more a
    tile, so the step takes 13.  With 7 decoding, 9 + 7 = two tiles would give 4.5 a tile against 16 / 3: the budget
    stays.  Outputs are the same as without the quantum."""
    s, runner = make(pages=64, budget=16, row_quantum=8, max_model_len=64)
    decoders = [req(i, 2, 12) for i in range(3)]
    for r in decoders:
        s.add_request(r)
    s.step()                                   # three short prompts, whole: 6 prompt tokens
    assert runner.batches[0] == [(0, 2, [1]), (1, 2, [1]), (2, 2, [1])]
    long = req(9, 40, 2)
    s.add_request(long)
    s.step()
    assert runner.batches[1] == [(0, 1, [0]), (1, 1, [0]), (2, 1, [0]), (9, 13, [])]        # 3 + 13 = 16 rows
    s.step()
    assert runner.batches[2][-1] == (9, 13, [])
    more = [req(20 + i, 2, 12) for i in range(4)]
    for r in more:
        s.add_request(r)
    s.step()                                   # the long prompt's 13, and of the four new ones what the cut budget leaves
    assert sum(n for _, n, _ in runner.batches[3]) % 8 == 0
    s.run_to_completion()
    for r in decoders + more + [long]:
        assert r.output_token_ids == expected_output(r.prompt_token_ids, r.sampling.max_tokens)
    # seven riders: the cut would leave 9 prompt tokens on two tiles, fewer a tile than 16 on three
    s2, runner2 = make(pages=64, budget=16, row_quantum=8, max_model_len=64)
    riders = [req(i, 2, 12) for i in range(7)]
    for r in riders:
        s2.add_request(r)
    s2.step()
    s2.add_request(req(9, 40, 2))
    s2.step()
    assert runner2.batches[1][-1] == (9, 16, [])
    # off: the budget as it is
    s3, runner3 = make(pages=64, budget=16, max_model_len=64)
    for r in [req(i, 2, 12) for i in range(3)]:
        s3.add_request(r)
    s3.step()
    s3.add_request(req(9, 40, 2))
    s3.step()
    assert runner3.batches[1][-1] == (9, 16, [])


def test_portions_down_to_one_token():
    s, runner = make(budget=1)
    a = req(0, 3, 2)
    s.add_request(a)
    s.run_to_completion()
    assert [b[0][1:] for b in runner.batches[:3]] == [(1, []), (1, []), (1, [0])]
    assert a.output_token_ids == expected_output(a.prompt_token_ids, 2)


def test_worst_case_admission_blocks_the_queue_in_order():
    s, runner = make(pages=6)     # page = 4 tokens
    big, small = req(0, 10, 10), req(1, 2, 2)         # 20 tokens = 5 pages; 4 tokens = 1 page
    blocked, tiny = req(2, 6, 6), req(3, 1, 1)        # 3 pages: does not fit beside the first two
    for r in (big, small, blocked, tiny):
        s.add_request(r)
    s.step()
    assert [b[0] for b in runner.batches[0]] == [0, 1]
    assert blocked.status == RequestStatus.WAITING and tiny.status == RequestStatus.WAITING   # no skipping ahead
    s.run_to_completion()
    assert all(r.finished for r in (big, small, blocked, tiny)) and s.stats["preemptions"] == 0
    assert blocked.output_token_ids == expected_output(blocked.prompt_token_ids, 6)


def test_finishing_on_eos_stop_and_at_prefill():
    s, _ = make()
    a = req(0, 4, 10)
    first = expected_output(a.prompt_token_ids, 3)
    a.eos_token_id = first[2]
    b = Request(1, a.prompt_token_ids, SamplingParams(max_tokens=10, stop_token_ids=(first[1],)))
    c = Request(2, a.prompt_token_ids, SamplingParams(max_tokens=10, ignore_eos=True), eos_token_id=first[0])
    d = Request(3, a.prompt_token_ids, SamplingParams(max_tokens=1))
    for r in (a, b, c, d):
        s.add_request(r)
    got = s.step()
    assert d in got and d.finished and d.finish_reason == "length"      # prefill alone finished it
    s.run_to_completion()
    assert a.output_token_ids == first and a.finish_reason == "stop"    # the eos token stays in the output
    assert b.output_token_ids == first[:2] and b.finish_reason == "stop"
    assert len(c.output_token_ids) == 10 and c.finish_reason == "length"


def test_pages_run_out_youngest_is_preempted_keeps_tokens_and_finishes_the_same():
    s, runner = make(pages=6, admission="optimistic")
    a, b = req(0, 7, 9), req(1, 6, 9)        # together they outgrow 6 pages of 4 tokens
    s.add_request(a); s.add_request(b)
    s.run_to_completion()
    assert s.stats["preemptions"] >= 1 and b.preemptions >= 1 and a.preemptions == 0
    assert a.output_token_ids == expected_output(a.prompt_token_ids, 9)
    assert b.output_token_ids == expected_output(b.prompt_token_ids, 9)
    rerun = [batch for batch in runner.batches for (rid, n, _) in batch if rid == 1 and n > 6]
    assert rerun, "the preempted request is run again from its prompt plus the tokens it had generated"
    assert runner.cache.free_pages() == [6]


def test_a_request_that_could_never_fit_is_refused_at_once():
    s, _ = make(pages=2)
    with pytest.raises(ValueError, match="could never finish"):
        s.add_request(req(0, 6, 6))
    with pytest.raises(ValueError, match="empty prompt"):
        s.add_request(Request(1, []))
    with pytest.raises(ValueError, match="vocabulary"):
        s.add_request(Request(2, [VOCAB]))
    with pytest.raises(ValueError, match="model length"):
        s.add_request(Request(3, [1] * 64))


def test_generation_stops_at_the_model_length():
    s, _ = make(pages=32)
    a = Request(0, [1] * 60, SamplingParams(max_tokens=50))
    s.add_request(a)
    s.run_to_completion()
    assert a.num_tokens == 64 and a.finish_reason == "length"


def test_cancel_frees_pages_wherever_the_request_is():
    s, runner = make(pages=8, budget=4)
    a, b = req(0, 10, 4), req(1, 3, 4)
    s.add_request(a); s.add_request(b)
    s.step()
    assert s.cancel(0) and a.finish_reason == "cancelled"
    assert s.cancel(1) and not s.cancel(7)
    assert runner.cache.free_pages() == [8] and not s.has_unfinished()


def test_max_num_seqs_bounds_live_requests():
    s, runner = make(pages=64, max_num_seqs=2)
    rs = [req(i, 3, 2) for i in range(5)]
    for r in rs:
        s.add_request(r)
    while s.has_unfinished():
        s.step()
        assert len(s.live) <= 2
    assert all(r.output_token_ids == expected_output(r.prompt_token_ids, 2) for r in rs)


def test_seeds_are_drawn_once_and_kept_over_preemption():
    s, _ = make(pages=6, admission="optimistic", seed=5)
    a, b = req(0, 7, 9), req(1, 6, 9, seed=1234)
    s.add_request(a); s.add_request(b)
    seed_a = a.seed
    s.run_to_completion()
    assert b.seed == 1234 and a.seed == seed_a and b.preemptions >= 1


# ---- pipelined scheduling: step k+1 is launched before the tokens of step k are read ----

def run_both(make_requests, **kw):
    out = []
    for pipelined in (False, True):
        s, runner = make(async_scheduling=pipelined, **kw)
        rs = make_requests()
        for r in rs:
            s.add_request(r)
        done = s.run_to_completion()
        assert sorted(r.request_id for r in done) == sorted(r.request_id for r in rs)     # each finishes once
        assert runner.cache.free_pages() == [kw.get("pages", 16)] and not s.has_unfinished()
        out.append((s, runner, rs))
    return out


def test_pipelined_steps_take_tokens_from_the_device_and_give_the_same_outputs():
    (s0, run0, plain), (s1, run1, piped) = run_both(lambda: [req(0, 5, 6), req(1, 9, 4), req(2, 3, 1)], pages=32)
    for a, b in zip(plain, piped):
        assert a.output_token_ids == b.output_token_ids == expected_output(a.prompt_token_ids, a.sampling.max_tokens)
        assert a.finish_reason == b.finish_reason == "length"
    assert sum(run0.from_device) == 0 and sum(run1.from_device) > 0
    assert run1.batches == run0.batches                  # ends that are known by count waste no step
    assert s1.stats["dropped_tokens"] == 0


def test_pipelined_returns_the_tokens_of_the_step_before():
    s, runner = make(async_scheduling=True)
    a = req(0, 5, 4)
    s.add_request(a)
    assert s.step() == [] and a.inflight == 1 and a.output_token_ids == []      # sampled, not read yet
    assert s.step() == [a] and len(a.output_token_ids) == 1 and a.inflight == 1
    assert runner.from_device == [0, 1]
    s.run_to_completion()
    assert a.output_token_ids == expected_output(a.prompt_token_ids, 4)


def test_pipelined_stop_token_costs_one_dropped_token_and_frees_the_pages():
    first = expected_output(req(0, 4).prompt_token_ids, 3)
    (s0, run0, plain), (s1, run1, piped) = run_both(
        lambda: [Request(0, req(0, 4).prompt_token_ids, SamplingParams(max_tokens=10, stop_token_ids=(first[1],))),
                 req(1, 6, 5)], pages=16)
    assert plain[0].output_token_ids == piped[0].output_token_ids == first[:2] and piped[0].finish_reason == "stop"
    assert plain[1].output_token_ids == piped[1].output_token_ids
    assert s1.stats["dropped_tokens"] == 1 and s0.stats["dropped_tokens"] == 0
    ran = [sum(1 for rid, _, _ in b if rid == 0) for b in run1.batches]
    assert sum(ran) == sum(1 for b in run0.batches for rid, _, _ in b if rid == 0) + 1   # it ran once more


def test_pipelined_with_budget_preemption_and_late_arrivals():
    def requests():
        return [req(0, 7, 9), req(1, 6, 9), req(2, 11, 3)]
    (s0, _, plain), (s1, run1, piped) = run_both(requests, pages=7, budget=5, admission="optimistic")
    assert s1.stats["preemptions"] >= 1
    for a, b in zip(plain, piped):
        assert a.output_token_ids == b.output_token_ids == expected_output(a.prompt_token_ids, a.sampling.max_tokens)


def test_pipelined_with_a_row_quantum_budget_and_preemption():
    """The cut of the budget to whole tiles of rows counts the requests that ride along; with tokens in flight those
    whose last token is in flight ride no more.  Outputs are what they are without pipelining and without the cut."""
    def requests():
        return [req(0, 7, 9), req(1, 6, 9), req(2, 23, 3), req(3, 5, 2)]
    (s0, run0, plain), (s1, run1, piped) = run_both(requests, pages=12, budget=9, admission="optimistic", row_quantum=4)
    for a, b in zip(plain, piped):
        assert a.output_token_ids == b.output_token_ids == expected_output(a.prompt_token_ids, a.sampling.max_tokens)
    # a step that took the cut has a multiple of four rows
    cut = [b for b in run0.batches if sum(n for _, n, _ in b) % 4 == 0 and any(n > 1 for _, n, _ in b) and any(n == 1 for _, n, _ in b)]
    assert cut, run0.batches


def test_pipelined_repetition_penalty_sees_every_earlier_token():
    s, _ = make(async_scheduling=True)
    a = Request(0, [3, 4, 5], SamplingParams(max_tokens=4, repetition_penalty=1.3))
    s.add_request(a)
    s.run_to_completion()
    assert a.output_token_ids == expected_output(a.prompt_token_ids, 4)
    for counters, seen in s.sampler.seen_at_launch:
        assert len(seen[0]) == len(set(a.output_token_ids[:counters[0]]))   # nothing in flight when it is sampled


def test_pipelined_cancel_with_a_token_in_flight():
    s, runner = make(async_scheduling=True)
    a, b = req(0, 5, 6), req(1, 4, 6)
    s.add_request(a); s.add_request(b)
    s.step(); s.step()
    assert a.inflight == 1 and s.cancel(0)
    s.run_to_completion()
    assert a.finish_reason == "cancelled" and len(a.output_token_ids) == 1
    assert b.output_token_ids == expected_output(b.prompt_token_ids, 6)
    assert runner.cache.free_pages() == [16] and s.stats["dropped_tokens"] == 1
