"""The sampling kernel against the plain statement of the reference's sampler
(tests/plain_gemma.py: penalise_repeats, kept_mask, sampling_distribution)."""
import pytest
import torch

import plain_gemma as plain
from wllm_b200.sampling import SamplingParams, uniform_from

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CASES = [
    SamplingParams(temperature=0.0),
    SamplingParams(temperature=0.8),
    SamplingParams(temperature=1.3, top_k=5),
    SamplingParams(temperature=0.7, top_p=0.6),
    SamplingParams(temperature=1.0, min_p=0.05),
    SamplingParams(temperature=0.9, top_k=40, top_p=0.9, min_p=0.01),
    SamplingParams(temperature=0.0, repetition_penalty=1.7),
    SamplingParams(temperature=1.1, top_p=0.8, repetition_penalty=1.3),
    SamplingParams(temperature=0.5, top_k=1),
    SamplingParams(temperature=2.0, top_p=0.05),      # rank 0 alone
]


def run(logits, params, counters, seeds, generated):
    from wllm_b200.sampling.sampler import Sampler
    return Sampler(DEV).sample(logits.to(DEV).clone(), params, counters, seeds, generated)


@pytest.mark.parametrize("V", [1000, 2513, 50001])
def test_rows_follow_the_plain_sampler(V):
    g = torch.Generator().manual_seed(V)
    rows = len(CASES) * 3
    logits = torch.randn(rows, V, generator=g) * 3.0
    params = [CASES[i % len(CASES)] for i in range(rows)]
    counters = [i * 7 % 13 for i in range(rows)]
    seeds = [1000 + i for i in range(rows)]
    generated = [set(torch.randint(0, V, (20,), generator=g).tolist()) for _ in range(rows)]
    tokens, logprobs = run(logits, params, counters, seeds, generated)
    for i, p in enumerate(params):
        probs, logp = plain.sampling_distribution(logits[i], p.temperature, p.top_k, p.top_p, p.min_p,
                                                  p.repetition_penalty, generated[i])
        tok = tokens[i]
        assert abs(logprobs[i] - float(logp[tok])) < 2e-4, (i, p)
        if p.temperature == 0.0:
            assert tok == int(probs.argmax())
            continue
        assert float(probs[tok]) > 0.0, f"row {i} {p}: token {tok} is filtered out by the plain sampler"
        cdf = probs.cumsum(0)
        u = uniform_from(seeds[i], counters[i])
        lo = float(cdf[tok - 1]) if tok > 0 else 0.0
        assert lo - 1e-5 <= u <= float(cdf[tok]) + 1e-5, (i, p, u, lo, float(cdf[tok]))


def test_a_row_does_not_depend_on_the_batch():
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(6, 4099, generator=g) * 2
    p = SamplingParams(temperature=0.9, top_k=50, top_p=0.95)
    together, _ = run(logits, [p] * 6, [3] * 6, list(range(6)), [set()] * 6)
    for i in range(6):
        alone, _ = run(logits[i:i + 1], [p], [3], [i], [set()])
        assert alone[0] == together[i]
    again, _ = run(logits, [p] * 6, [4] * 6, list(range(6)), [set()] * 6)
    assert again != together           # another output place draws another number


def test_draws_follow_the_distribution():
    probs = torch.tensor([0.5, 0.3, 0.15, 0.05])
    logits = probs.log().repeat(4000, 1)
    p = SamplingParams(temperature=1.0)
    tokens, _ = run(logits, [p] * 4000, list(range(4000)), [77] * 4000, [set()] * 4000)
    freq = torch.bincount(torch.tensor(tokens), minlength=4).float() / 4000
    assert float((freq - probs).abs().max()) < 0.03


def test_greedy_ties_take_the_lowest_id():
    logits = torch.zeros(2, 300)
    logits[0, [17, 250]] = 5.0
    logits[1, 299] = 1.0
    tokens, _ = run(logits, [SamplingParams()] * 2, [0, 0], [0, 0], [set(), set()])
    assert tokens == [17, 299]


@pytest.mark.parametrize("V", [31, 1000, 256000])
def test_all_greedy_batches_take_the_two_stage_path(V):
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(5, V, generator=g) * 4.0
    logits[2, V - 1] = 50.0                      # the last token of the last chunk
    logits[3, 0] = logits[3, V // 2] = 60.0      # equal maxima in different chunks: the lower id wins
    tokens, logprobs = run(logits, [SamplingParams()] * 5, [0] * 5, [0] * 5, [set()] * 5)
    want = torch.log_softmax(logits.double(), dim=-1)
    assert tokens == logits.argmax(-1).tolist() and tokens[2] == V - 1 and tokens[3] == 0
    for i, t in enumerate(tokens):
        assert abs(logprobs[i] - float(want[i, t])) < 2e-4
