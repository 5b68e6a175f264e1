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
def test_all_greedy_batches_need_no_options(V):
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(5, V, generator=g) * 4.0
    logits[2, V - 1] = 50.0                      # the last token of the last chunk
    logits[3, 0] = logits[3, V // 2] = 60.0      # equal maxima in different chunks: the lower id wins
    tokens, logprobs = run(logits, [SamplingParams()] * 5, [0] * 5, [0] * 5, [set()] * 5)
    want = torch.log_softmax(logits.double(), dim=-1)
    assert tokens == logits.argmax(-1).tolist() and tokens[2] == V - 1 and tokens[3] == 0
    for i, t in enumerate(tokens):
        assert abs(logprobs[i] - float(want[i, t])) < 2e-4


def check_against_plain(logits, params, counters, seeds, generated, tokens, logprobs):
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


def test_a_vocabulary_of_256000_with_every_filter():
    """The size the engine serves: rows cut into 32 chunks each, three selection passes."""
    V = 256000
    g = torch.Generator().manual_seed(5)
    rows = len(CASES) + 2
    logits = torch.randn(rows, V, generator=g) * 2.5
    logits[:, 1234] += 9.0                       # a peaked row, as a model's is
    params = CASES + [SamplingParams(temperature=1.0, top_k=V - 1), SamplingParams(temperature=1.5, top_p=0.999)]
    counters = [i * 5 % 11 for i in range(rows)]
    seeds = [2 ** 40 + i for i in range(rows)]
    generated = [set(torch.randint(0, V, (300,), generator=g).tolist()) | {1234} for _ in range(rows)]
    tokens, logprobs = run(logits, params, counters, seeds, generated)
    check_against_plain(logits, params, counters, seeds, generated, tokens, logprobs)


def kept_by_kernel(logits_row, p, draws=400):
    """Ids that the kernel draws for one row under `draws` different counters."""
    rows = logits_row.repeat(draws, 1)
    tokens, _ = run(rows, [p] * draws, list(range(draws)), [9] * draws, [set()] * draws)
    return set(tokens)


def test_equal_values_at_a_threshold_stay_or_go_together():
    """Where a filter's edge falls among equal values, a sort cuts among them by its own order (the plain
    sampler's stable sort by id); the kernel's thresholds are values, so equals stay or go together."""
    V = 3000
    logits = torch.full((V,), -12.0)
    leaders, runners = [5, 700, 1500, 2999], [6, 800, 1600]
    logits[leaders] = 3.0
    logits[runners] = 2.0
    both = set(leaders) | set(runners)
    # top-k = 2 cuts among the four leaders: all four stay (the k-th largest value is 3.0), no runner-up does
    assert kept_by_kernel(logits, SamplingParams(temperature=1.0, top_k=2)) == set(leaders)
    # top-k = 5 reaches into the runners-up: all three come along
    assert kept_by_kernel(logits, SamplingParams(temperature=1.0, top_k=5), 800) == both
    # top-p: the leaders hold 0.78 of the mass, leaders and runners-up 0.9998
    z = 4 * torch.e ** 3 + 3 * torch.e ** 2 + (V - 7) * torch.e ** -12
    assert 4 * torch.e ** 3 / z < 0.8 < 0.9 < (4 * torch.e ** 3 + 3 * torch.e ** 2) / z < 0.9999
    assert kept_by_kernel(logits, SamplingParams(temperature=1.0, top_p=0.9)) == set(leaders)
    assert kept_by_kernel(logits, SamplingParams(temperature=1.0, top_p=0.9999), 800) == both
    # a budget below the leaders' mass: rank 0 always stays, and its equals with it
    assert kept_by_kernel(logits, SamplingParams(temperature=1.0, top_p=0.5)) == set(leaders)
    # min-p just above and just below e^-1, the runners-up's ratio to the leaders
    assert kept_by_kernel(logits, SamplingParams(temperature=1.0, min_p=0.40)) == set(leaders)
    assert kept_by_kernel(logits, SamplingParams(temperature=1.0, min_p=0.35), 800) == both


def test_a_row_of_equal_logits_draws_from_everything():
    V = 5000
    tokens = kept_by_kernel(torch.zeros(V), SamplingParams(temperature=0.7, top_k=3, top_p=0.2), 600)
    assert len(tokens) > 500 and min(tokens) < 100 and max(tokens) > V - 100


def test_tokens_do_not_depend_on_how_rows_are_cut_into_chunks():
    """Up to 8 rows are cut into 64 chunks each, more rows into 32; sums of masses are integers, so the same
    row draws the same token either way, and one sampler serves calls of every kind in turn."""
    from wllm_b200.sampling.sampler import Sampler
    V = 70001
    g = torch.Generator().manual_seed(3)
    base = (torch.randn(130, V, generator=g) * 3.0).to(DEV)
    params = [CASES[i % len(CASES)] for i in range(130)]
    counters, seeds = [i % 17 for i in range(130)], [50 + i for i in range(130)]
    generated = [set(range(i, i + 40)) for i in range(130)]
    sampler = Sampler(DEV)

    def draw(n):
        return sampler.sample(base[:n].clone(), params[:n], counters[:n], seeds[:n], generated[:n])
    many, many_lp = draw(130)
    nine, _ = draw(9)
    assert nine == many[:9]
    for i in range(len(CASES)):
        tok, lp = sampler.sample(base[i:i + 1].clone(), [params[i]], [counters[i]], [seeds[i]], [generated[i]])
        assert tok[0] == many[i] and abs(lp[0] - many_lp[i]) < 1e-5
    again, _ = draw(130)
    assert again == many
    check_against_plain(base[:20].cpu(), params[:20], counters[:20], seeds[:20], generated[:20], many[:20], many_lp[:20])


def test_a_vocabulary_too_long_for_the_register_and_shared_memory_paths():
    """600,001 logits a row: chunks longer than a thread block keeps in registers, segments longer than
    the draw stages in shared memory, and rows that do not start on a 16-byte boundary."""
    V = 600001
    g = torch.Generator().manual_seed(8)
    params = [SamplingParams(temperature=0.9, top_k=30, top_p=0.9), SamplingParams(temperature=1.2, min_p=0.02),
              SamplingParams(temperature=0.0), SamplingParams(temperature=0.8)]
    rows = len(params)
    logits = torch.randn(rows, V, generator=g) * 3.0
    logits[:, V - 1] += 6.0
    counters, seeds, generated = [1, 2, 3, 4], [11, 12, 13, 14], [set()] * rows
    tokens, logprobs = run(logits, params, counters, seeds, generated)
    check_against_plain(logits, params, counters, seeds, generated, tokens, logprobs)
    many, _ = run(logits.repeat(3, 1), params * 3, counters * 3, seeds * 3, generated * 3)     # 12 rows: 32 chunks each
    assert many == tokens * 3
