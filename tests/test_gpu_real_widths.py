"""The engine at the real layer widths of Gemma-2B and Gemma-7B (two layers each, the whole
256,000-token vocabulary, random weights): logits under several ways of cutting against the
plain implementation run in float32 on the host, in 32-bit (also bit-equal across cuts) and
in bfloat16.  These are the sizes at which index arithmetic, tile tails and split plans of
the kernels differ from the tiny configurations."""
import os

import pytest
import torch
from safetensors.torch import load_file

import plain_gemma as plain
import traces
from helpers import max_diff

pytestmark = pytest.mark.gpu

SHAPES = {
    "2b": dict(hidden_size=2048, num_attention_heads=8, num_key_value_heads=1, head_dim=256, intermediate_size=16384),
    "7b": dict(hidden_size=3072, num_attention_heads=16, num_key_value_heads=16, head_dim=256, intermediate_size=24576),
}


def config(name):
    return dict(architectures=["GemmaForCausalLM"], model_type="gemma", num_hidden_layers=2, vocab_size=256000,
                max_position_embeddings=8192, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                **SHAPES[name])


@pytest.fixture(scope="module", params=["2b", "7b"])
def model(request, tmp_path_factory):
    from wllm_b200.weights import write_random_model
    name = request.param
    cfg = config(name)
    folder = write_random_model(str(tmp_path_factory.mktemp(name) / "m"), cfg, seed=3)
    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    g = torch.Generator().manual_seed(2)
    reqs = {"a": torch.randint(0, cfg["vocab_size"], (150,), generator=g).tolist(),
            "b": torch.randint(0, cfg["vocab_size"], (70,), generator=g).tolist(),
            "c": torch.randint(0, cfg["vocab_size"], (3,), generator=g).tolist()}
    # the plain implementation's logits at a handful of places per request (the head is 256,000 wide)
    wanted = {"a": [0, 1, 63, 64, 100, 149], "b": [0, 15, 16, 69], "c": [0, 2]}
    ref = {}
    for rid, toks in reqs.items():
        logits = plain.forward(toks, w, cfg)
        for p in wanted[rid]:
            ref[(rid, p)] = logits[p].clone()
    return name, folder, reqs, ref


def run(folder, dtype, steps, keys):
    from test_gpu_replay import gpu_runner
    pages = -(-traces.peak_tokens(steps) // 16)
    rows = traces.run_in_process(gpu_runner(folder, dtype, 16, pages), steps)
    return {k: rows[k] for k in keys}


def cuts(reqs):
    return {"whole": traces.whole(reqs), "tail": traces.tail_singly(reqs, tail=8),
            "portions": traces.portions(reqs, sizes=(64, 7, 2, 33, 70, 1)), "mixed": traces.mixed(reqs, seed=4, decode_tail=5)}


def test_32bit_matches_plain_and_is_bit_equal_across_cuts(model):
    name, folder, reqs, ref = model
    first = None
    for cut, steps in cuts(reqs).items():
        rows = run(folder, torch.float32, steps, ref.keys())
        assert max_diff(rows, ref) < 2e-4, (name, cut)       # logits of order 1 over sums of 16k-24k terms
        if first is None:
            first = rows
        else:
            bad = sorted(k for k in first if not torch.equal(first[k], rows[k]))
            assert not bad, f"{name} {cut}: first differing (request, position) {bad[0]}"


def test_bfloat16_matches_plain_under_every_cut(model):
    """Logits of up to 19 after two layers at either width; the largest difference observed under any cut is 0.022
    (Gemma-2B widths) and 0.034 (7B): 0.12 % and 0.18 % of the scale, from bfloat16 operands over sums of 16k to
    24k terms.  The bound is twice the larger, relative to the scale."""
    name, folder, reqs, ref = model
    scale = max(float(r.abs().max()) for r in ref.values())
    for cut, steps in cuts(reqs).items():
        rows = run(folder, torch.bfloat16, steps, ref.keys())
        worst = max_diff(rows, ref)
        assert worst < 0.004 * max(1.0, scale), f"{name} {cut}: largest difference {worst:.3e} on logits of up to {scale:.1f}"


def test_steps_queued_back_to_back_see_their_own_index_arrays(model):
    """Whole prompts stepped one after the other with no synchronisation in between and their logits dropped
    at once: the host builds and sends the next step's index arrays while the step before still runs, and a
    tensor freed on the host is still in use on the device.  The last step's logits are what a lone step gives.
    (A staging buffer that the copy stream wrote too early once showed here as an illegal address.)"""
    from test_gpu_replay import gpu_runner
    from wllm_b200.engine import StepEntry
    name, folder, reqs, ref = model
    runner = gpu_runner(folder, torch.bfloat16, 16, 64)
    for i in range(6):
        rc = runner.cache.open(f"warm{i}")
        runner.step([StepEntry(rc, reqs["a"], [len(reqs["a"]) - 1])])       # result dropped, nothing waited for
        runner.cache.close(rc)
    rc = runner.cache.open("last")
    got = runner.step([StepEntry(rc, reqs["b"], [69])])[0].float().cpu()
    lone = gpu_runner(folder, torch.bfloat16, 16, 64)
    want = lone.step([StepEntry(lone.cache.open("x"), reqs["b"], [69])])[0].float().cpu()
    assert torch.equal(got, want)
    scale = max(float(r.abs().max()) for r in ref.values())
    assert float((got.double() - ref[("b", 69)].double()).abs().max()) < 0.004 * max(1.0, scale)
