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


@pytest.mark.parametrize("dtype,margin", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_scarce_pages_with_poisoned_pages(folders, dtype, margin):
    """The same shortage with pages that hold NaN until written and again once given back (a preempted
    request's pages go to its neighbours at once): every token is still what the plain implementation draws."""
    prompts = prompts_of("A", (30, 41, 22, 35), seed=4)
    sp = SamplingParams(temperature=0.7, seed=9, max_tokens=40, ignore_eos=True)
    engine = llm(folders["A"], dtype=dtype, block_size=16, num_blocks=12, admission="optimistic",
                 chunked_prefill_tokens=24, poison_pages=True)
    outs = engine.generate(prompts, sp)
    assert engine.stats["preemptions"] >= 1 and engine.runner.cache.free_pages() == [12]
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 40
        check_against_plain("A", folders["A"], p, o.token_ids, sp, sp.seed, margin)


def test_a_kernel_that_gave_up_waiting_stops_generation(folders):
    """The status word that bounded waits in the tensor-core kernels set travels back with every step's sampled
    ids; a step that finds it set raises instead of handing on tokens made from partial results, and clears it."""
    from wllm_b200.kernels import KernelError, ops
    engine = llm(folders["A"], dtype="bfloat16")
    ops._status_word(engine.engine_config.device).fill_(21)
    with pytest.raises(KernelError, match="gave up waiting.*decode attention"):
        engine.generate([[5, 6, 7]], SamplingParams(max_tokens=3, ignore_eos=True))
    assert ops.tc_gemm_status(engine.engine_config.device) == 0
    outs = llm(folders["A"], dtype="bfloat16", async_scheduling=True).generate([[5, 6, 7]],
                                                                             SamplingParams(max_tokens=3, ignore_eos=True))
    assert len(outs[0].token_ids) == 3


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


@pytest.mark.parametrize("dtype,margin", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_captured_steps_across_table_widths_batch_buckets_and_a_regrown_index_buffer(folders, dtype, margin):
    """Eight requests that grow from one to three pages to more than sixteen (captures for tables of 8, 16 and
    32 pages) and end one after the other (captures for 8, 6, 4, 3, 2 and 1 requests).  Then, on the same
    engine, three long prompts whole in one step: their index arrays outgrow the buffer that the captures
    point into, which drops every capture, and the decode steps behind them are captured anew.  In 32-bit
    the tokens are the eager engine's; in both precisions they are what the plain implementation draws."""
    lengths, news = (5, 40, 77, 3, 21, 9, 60, 33), (300, 33, 150, 12, 250, 80, 40, 200)
    prompts = prompts_of("B", lengths, seed=6)
    sps = [SamplingParams(temperature=0.8, seed=70 + i, max_tokens=n, ignore_eos=True) for i, n in enumerate(news)]
    kw = dict(dtype=dtype, block_size=16, num_blocks=240, max_num_seqs=16)
    eager, graphed = llm(folders["B"], **kw), llm(folders["B"], cuda_graphs=True, **kw)
    want, outs = eager.generate(prompts, sps), graphed.generate(prompts, sps)
    keys = set(graphed.runner._graphs)
    assert {w for _, w in keys} >= {8, 16, 32}, keys
    assert {b for b, _ in keys} >= {1, 2, 3, 4, 6, 8}, keys
    meta = graphed.runner._meta.numel()
    long_prompts = prompts_of("B", (480, 470, 460), seed=7)
    sp2 = SamplingParams(temperature=0.8, seed=90, max_tokens=20, ignore_eos=True)
    want += eager.generate(long_prompts, sp2)
    outs += graphed.generate(long_prompts, sp2)
    assert graphed.runner._meta.numel() > meta, "the long prompts were meant to outgrow the index buffer"
    assert graphed.runner._graphs and all(rec["meta"] is graphed.runner._meta for rec in graphed.runner._graphs.values())
    assert graphed.runner.graph_launches > 0 and eager.runner.graph_launches == 0
    if dtype == "float32":
        assert [o.token_ids for o in outs] == [o.token_ids for o in want]
    for p, o, sp in zip(prompts + long_prompts, outs, sps + [sp2] * 3):
        assert len(o.token_ids) == sp.max_tokens
        check_against_plain("B", folders["B"], p, o.token_ids, sp, sp.seed, margin)


def test_the_command_line_generates_what_the_python_entry_point_does(folders):
    """`python -m wllm_b200 --model DIR ...` in a process of its own: its JSON lines carry the tokens of
    LLM.generate with the same options (random prompts from the same seed, portions of 16, captured graphs)."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "wllm_b200", "--model", folders["B"], "--dtype", "float32", "--block-size", "32",
           "--num-blocks", "24", "--prompt-lens", "5,40,77", "--prompt-seed", "3", "--prompt-ids", "7,8,9",
           "--cuda-graphs", "--chunked-prefill-tokens", "16", "--temperature", "0.7", "--top-k", "40", "--seed", "11",
           "--max-tokens", "12", "--ignore-eos", "--log-level", "WARNING"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=root)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(x) for x in proc.stdout.splitlines() if x.startswith("{")]
    g = torch.Generator().manual_seed(3)
    prompts = [[7, 8, 9]] + [torch.randint(0, CONFIGS["B"]["vocab_size"], (n,), generator=g).tolist() for n in (5, 40, 77)]
    sp = SamplingParams(temperature=0.7, top_k=40, seed=11, max_tokens=12, ignore_eos=True)
    outs = llm(folders["B"], dtype="float32", block_size=32, num_blocks=24, chunked_prefill_tokens=16,
               cuda_graphs=True).generate(prompts, sp)
    assert [x["token_ids"] for x in lines] == [o.token_ids for o in outs]
    assert [x["prompt_tokens"] for x in lines] == [3, 5, 40, 77] and all(x["finish_reason"] == "length" for x in lines)


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
