"""Generation through the Python entry point against the plain implementation: greedy
(tiny A: prompts of 7, 19 and 33 tokens, 16 tokens each), seeded temperature sampling with
prompts cut into portions of 16 beside decoding requests (tiny B: prompts of 1, 4, 50, 64
and 120 tokens, 24 tokens each), scarce pages with preemption, long decoding and the first
tokens of a sequence."""
import pytest
import torch

import plain_gemma as plain
import traces
from helpers import folder_weights, make_folder, max_diff, plain_rows, random_requests
from tiny_configs import CONFIGS
from wllm_b200.sampling import SamplingParams, uniform_from

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: make_folder(tmp_path_factory.mktemp("g"), n) for n in ("A", "B")}


def llm(folder, **kw):
    from wllm_b200 import LLM
    return LLM(folder, **kw)


def prompts_of(name, lengths, seed=1):
    return list(random_requests(name, lengths, seed).values())


def check_against_plain(name, folder, prompt, out, sp, seed, margin):
    """Every generated token is what the plain implementation picks at that place, given the
    tokens before it: the arg-max (within `margin` of the top logit, which is 0 for float32
    and covers a near-tie under bfloat16), or the inverse-CDF draw for (seed, place)."""
    w = folder_weights(folder)
    logits = plain.forward(prompt + out, w, CONFIGS[name])
    for i, tok in enumerate(out):
        row = logits[len(prompt) + i - 1]
        if sp.temperature == 0.0:
            assert float(row.max() - row[tok]) <= margin, (i, tok, int(row.argmax()))
        else:
            probs, _ = plain.sampling_distribution(row, sp.temperature, sp.top_k, sp.top_p, sp.min_p)
            cdf, u = probs.cumsum(0), uniform_from(seed, i)
            lo = float(cdf[tok - 1]) if tok > 0 else 0.0
            assert lo - margin - 1e-5 <= u <= float(cdf[tok]) + margin + 1e-5, (i, tok, u)


@pytest.mark.parametrize("dtype,margin", [("float32", 0.0), ("bfloat16", 2e-2)])
def test_greedy_tiny_a(folders, dtype, margin):
    prompts = prompts_of("A", (7, 19, 33))
    sp = SamplingParams(max_tokens=16, ignore_eos=True)
    outs = llm(folders["A"], dtype=dtype, block_size=16, num_blocks=24).generate(prompts, sp)
    w = folder_weights(folders["A"])
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 16 and o.finish_reason == "length"
        if dtype == "float32":
            assert o.token_ids == plain.greedy(p, w, CONFIGS["A"], 16)
        check_against_plain("A", folders["A"], p, o.token_ids, sp, 0, margin)


@pytest.mark.parametrize("dtype,margin", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_seeded_temperature_tiny_b_portions_mixed_with_decoding(folders, dtype, margin):
    prompts = prompts_of("B", (1, 4, 50, 64, 120))
    sps = [SamplingParams(temperature=0.8, seed=40 + i, max_tokens=24, ignore_eos=True) for i in range(5)]
    engine = llm(folders["B"], dtype=dtype, block_size=32, num_blocks=16, chunked_prefill_tokens=16)
    outs = engine.generate(prompts, sps)
    assert engine.stats["steps"] > 24       # the 120-token prompt alone takes 8 portions
    for p, o, sp in zip(prompts, outs, sps):
        assert len(o.token_ids) == 24
        check_against_plain("B", folders["B"], p, o.token_ids, sp, sp.seed, margin)
    if dtype == "float32":    # alone and whole, each request draws the same tokens
        for p, o, sp in zip(prompts, outs, sps):
            alone = llm(folders["B"], dtype=dtype, block_size=32, num_blocks=16).generate([p], sp)[0]
            assert alone.token_ids == o.token_ids


def test_scarce_pages_preempt_and_change_nothing(folders):
    prompts = prompts_of("A", (30, 41, 22, 35), seed=4)
    sp = SamplingParams(temperature=0.7, top_k=20, seed=9, max_tokens=40, ignore_eos=True)
    roomy = llm(folders["A"], dtype="float32", block_size=16, num_blocks=64).generate(prompts, sp)
    tight_engine = llm(folders["A"], dtype="float32", block_size=16, num_blocks=12, admission="optimistic",
                       chunked_prefill_tokens=24)
    tight = tight_engine.generate(prompts, sp)
    assert tight_engine.stats["preemptions"] >= 1 and tight_engine.stats["pages_high_water"] == [12]
    assert [o.token_ids for o in tight] == [o.token_ids for o in roomy]
    assert tight_engine.runner.cache.free_pages() == [12]


def test_eos_and_stop_ids_end_a_request(folders):
    p = prompts_of("A", (9,))[0]
    sp = dict(temperature=1.5, seed=3, max_tokens=12)
    base = llm(folders["A"], dtype="float32").generate([p], SamplingParams(ignore_eos=True, **sp))[0].token_ids
    cut = next(i for i in range(2, 12) if base[i] not in base[:i])     # a token that appears there first
    out = llm(folders["A"], dtype="float32").generate([p], SamplingParams(stop_token_ids=(base[cut],), **sp))[0]
    assert out.token_ids == base[:cut + 1] and out.finish_reason == "stop"
    from wllm_b200 import LLM
    engine = LLM(folders["A"], dtype="float32")
    engine.eos_token_id = base[cut]
    out = engine.generate([p], SamplingParams(**sp))[0]
    assert out.token_ids == base[:cut + 1] and out.finish_reason == "stop"     # the eos token stays in the output


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 2e-2)])
def test_long_decoding(folders, dtype, tol):
    """Eight tokens at once, then nearly five hundred one by one, up to the model's last position."""
    from test_gpu_replay import gpu_runner
    reqs = random_requests("B", (500,), seed=8)
    steps = traces.tail_singly(reqs, tail=492)
    runner = gpu_runner(folders["B"], torch.float32 if dtype == "float32" else torch.bfloat16, 32, 16)
    rows = traces.run_in_process(runner, steps)
    assert max_diff(rows, plain_rows(folders["B"], "B", reqs)) < tol


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 2e-2)])
def test_first_tokens_of_a_sequence(folders, dtype, tol):
    from test_gpu_replay import gpu_runner
    reqs = random_requests("A", (1, 2, 3, 3), seed=2)
    for steps in (traces.whole(reqs), traces.tail_singly(reqs, tail=2), traces.mixed(reqs, seed=1, decode_tail=3)):
        runner = gpu_runner(folders["A"], torch.float32 if dtype == "float32" else torch.bfloat16, 16, 4)
        assert max_diff(traces.run_in_process(runner, steps), plain_rows(folders["A"], "A", reqs)) < tol


def test_the_engine_refuses_to_run_without_cuda_or_with_bad_ids(folders):
    from wllm_b200.kernels import KernelBuildError
    from wllm_b200.engine import build_model
    with pytest.raises(KernelBuildError, match="CUDA device only"):
        build_model(folders["A"], torch.float32, "cpu")
    engine = llm(folders["A"], dtype="float32")
    with pytest.raises(ValueError, match="vocabulary"):
        engine.generate([[5, 512]])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_decode_steps_change_nothing(folders, dtype):
    """Five requests that end at different lengths: the captured steps serve 5 in a capture for 6 (one request
    that brings no token is appended), then 4, 3, 2 and 1."""
    prompts = prompts_of("B", (5, 40, 77, 3, 21), seed=6)
    sp = [SamplingParams(temperature=0.9, seed=5, max_tokens=n, ignore_eos=True) for n in (40, 33, 40, 12, 25)]
    kw = dict(dtype=dtype, block_size=32, num_blocks=24, chunked_prefill_tokens=32)
    plain_run = llm(folders["B"], **kw).generate(prompts, sp)
    graphed = llm(folders["B"], cuda_graphs=True, **kw)
    outs = graphed.generate(prompts, sp)
    assert graphed.runner.graph_launches > 0
    assert [o.token_ids for o in outs] == [o.token_ids for o in plain_run]


@pytest.mark.parametrize("graphs", [False, True])
def test_pipelined_scheduling_changes_no_token(folders, graphs):
    """Steps launched before the host has read the tokens of the step before (decode entries take their
    token from the device): the same tokens as step by step, with stop ids, scarce pages and penalties."""
    prompts = prompts_of("B", (5, 40, 77, 3), seed=6)
    base = dict(temperature=0.9, seed=5, max_tokens=40)
    free_run = llm(folders["B"], dtype="float32", block_size=32, num_blocks=24).generate(
        prompts, SamplingParams(ignore_eos=True, **base))
    stop = free_run[1].token_ids[17]
    sps = [SamplingParams(ignore_eos=True, **base), SamplingParams(stop_token_ids=(stop,), **base),
           SamplingParams(ignore_eos=True, repetition_penalty=1.2, **base), SamplingParams(max_tokens=1)]
    kw = dict(dtype="float32", block_size=32, num_blocks=9, chunked_prefill_tokens=32, admission="optimistic",
              cuda_graphs=graphs)
    stepwise = llm(folders["B"], **kw).generate(prompts, sps)
    engine = llm(folders["B"], async_scheduling=True, **kw)
    piped = engine.generate(prompts, sps)
    assert [o.token_ids for o in piped] == [o.token_ids for o in stepwise]
    assert [o.finish_reason for o in piped] == [o.finish_reason for o in stepwise]
    assert piped[1].finish_reason == "stop" and piped[1].token_ids[-1] == stop
    assert [o.logprobs for o in piped] == [o.logprobs for o in stepwise]
    assert engine.runner.cache.free_pages() == [9] and not engine.has_unfinished()
    if graphs:
        assert engine.runner.graph_launches > 0


def test_pipelined_scheduling_bfloat16_against_plain(folders):
    prompts = prompts_of("A", (7, 19, 33))
    sp = SamplingParams(max_tokens=16, ignore_eos=True)
    outs = llm(folders["A"], dtype="bfloat16", block_size=16, num_blocks=24, async_scheduling=True,
               cuda_graphs=True).generate(prompts, sp)
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 16
        check_against_plain("A", folders["A"], p, o.token_ids, sp, 0, 2e-2)
