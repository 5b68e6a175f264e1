"""The engine on the GPU against the plain implementation, for every way of cutting the
same requests into steps: whole; most in one step and the last 32 tokens singly;
portions of changing size down to two tokens; and mixed, up to four live requests with
so few pages that they are used again.  In 32-bit and in bfloat16, on both tiny
configurations, in process and once through bin/trace_run."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import traces
from helpers import make_folder, max_diff, plain_rows, random_requests
from tiny_configs import CONFIGS, PAGE_SIZES

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = {"A": (7, 19, 33, 70, 41, 12, 90, 55, 66, 100), "B": (1, 4, 50, 64, 120, 37, 81, 2, 130, 77)}
# float32: kernels and plain implementation differ in summation order only.
# bfloat16: operands of every product are rounded to 8 bits of mantissa.  On these seeds the logits reach 1.6
# (tiny A) and 2.4 (tiny B) with a standard deviation near 0.2, and the largest difference observed under any
# cut is 1.6e-3 (A) and 1.9e-3 (B); the bound is twice the larger one.
TOL = {torch.float32: 3e-5, torch.bfloat16: 4e-3}
MODES = {"whole": traces.whole, "tail": traces.tail_singly, "portions": traces.portions,
         "mixed": lambda r: traces.mixed(r, seed=3)}


@pytest.fixture(scope="module")
def setups(tmp_path_factory):
    out = {}
    for name in ("A", "B"):
        folder = make_folder(tmp_path_factory.mktemp("m"), name)
        reqs = random_requests(name, LENGTHS[name], seed=5)
        out[name] = (folder, reqs, plain_rows(folder, name, reqs))
    return out


def gpu_runner(folder, dtype, page_size, pages, poison=False):
    from wllm_b200.config import EngineConfig
    from wllm_b200.engine import build_model, build_runner
    eng = EngineConfig(dtype=dtype, block_size=page_size, max_num_seqs=8)
    return build_runner(build_model(folder, eng.dtype, eng.device), eng, num_pages=pages, poison_pages=poison)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("poison", [False, True])
def test_every_cut_matches_plain(setups, dtype, name, mode, poison):
    """`poison`: pages hold NaN until a token is written there and again once they are given back, so a kernel
    that lets a slot past a request's keys, or a page of a request that ended, into its sums shows as NaN."""
    folder, reqs, ref = setups[name]
    steps = MODES[mode](reqs)
    ps = PAGE_SIZES[name]
    pages = -(-traces.peak_tokens(steps) // ps)
    runner = gpu_runner(folder, dtype, ps, pages, poison)
    rows = traces.run_in_process(runner, steps)
    worst = max_diff(rows, ref)
    assert worst < TOL[dtype], f"largest difference from the plain implementation {worst:.3e} (bound {TOL[dtype]:.0e})"
    assert runner.cache.free_pages() == [pages]
    if mode == "mixed":
        assert runner.cache.groups[0].pool.takes > pages, "the trace must use pages again"


@pytest.mark.parametrize("name", ["A", "B"])
def test_32bit_logits_do_not_depend_on_the_cut_at_all(setups, name):
    """In the 32-bit path every reduction has a fixed order per row, so the four traces
    agree bit for bit; any difference is a fault of the cache or the batch."""
    folder, reqs, _ = setups[name]
    ps = PAGE_SIZES[name]
    base = None
    for mode, make in MODES.items():
        steps = make(reqs)
        runner = gpu_runner(folder, torch.float32, ps, -(-traces.peak_tokens(steps) // ps))
        rows = traces.run_in_process(runner, steps)
        if base is None:
            base = rows
            continue
        bad = [k for k in base if not torch.equal(base[k], rows[k])]
        assert not bad, f"{mode}: first differing (request, position): {sorted(bad)[0]}"


def _cached_rows(runner, rc, n):
    """[layers, k|v, n, kv_heads, head_dim]: what the pages hold for the first n tokens of a live request."""
    ps = runner.cache.page_size
    pages = torch.tensor([rc.tables[0][p // ps] for p in range(n)], device="cuda")
    offs = torch.tensor([p % ps for p in range(n)], device="cuda")
    # (two index arrays apart from each other put their common axis first)
    return runner.cache.groups[0].pages[:, :, pages, :, offs, :].permute(1, 2, 0, 3, 4).float().cpu()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B"])
def test_pages_hold_the_same_keys_and_values_however_the_prompt_was_cut(setups, dtype, name):
    """The cache's contents, not only the logits: after a prompt went in whole, in portions down to one token,
    and token by token at its end, every layer's pages hold the same rotated keys and values at the request's
    slots (bit for bit in 32-bit), layer 0's are what the plain formulas give, and the slots behind the
    prompt's end were never written (the pools start as NaN here).  The reference looks at its cache after a
    chunked prefill the same way (tests/test_chunked_prefill.py:71-81)."""
    import plain_gemma as plain
    from helpers import folder_weights
    from wllm_b200.engine import StepEntry
    folder, reqs, _ = setups[name]
    cfg, ps = CONFIGS[name], PAGE_SIZES[name]
    rid, toks = max(reqs.items(), key=lambda kv: len(kv[1]))
    n = len(toks)
    held = []
    for cut in (traces.whole, traces.portions, lambda r: traces.tail_singly(r, tail=9)):
        steps = cut({rid: toks})
        runner = gpu_runner(folder, dtype, ps, -(-n // ps) + 2, poison=True)
        rc = runner.cache.open(rid)
        for s in steps:
            runner.step([StepEntry(rc, s["entries"][0]["tokens"], [])])
        held.append(_cached_rows(runner, rc, n))
        last, used = rc.tables[0][-1], n - (len(rc.tables[0]) - 1) * ps
        tail = runner.cache.groups[0].pages[:, :, last, :, used:, :]
        assert bool(torch.isnan(tail.float()).all()), "slots behind the prompt's end were written"
    exact = dtype == torch.float32
    for other in held[1:]:
        if exact:
            assert torch.equal(other, held[0])
        else:
            torch.testing.assert_close(other, held[0], rtol=0, atol=4e-3)
    w = folder_weights(folder)
    x = plain.rms_norm(plain.embed(torch.tensor(toks), w["model.embed_tokens.weight"], cfg["hidden_size"]),
                       w["model.layers.0.input_layernorm.weight"], cfg["rms_norm_eps"])
    nkv, hd = cfg["num_key_value_heads"], cfg["head_dim"]
    cos, sin = plain.rope_tables(torch.arange(n), hd, cfg["rope_theta"])
    k = plain.apply_rope((x @ w["model.layers.0.self_attn.k_proj.weight"].T).view(n, nkv, hd), cos, sin)
    v = (x @ w["model.layers.0.self_attn.v_proj.weight"].T).view(n, nkv, hd)
    tol = 2e-5 if exact else 4e-3
    torch.testing.assert_close(held[0][0, 0], k, rtol=0, atol=tol)
    torch.testing.assert_close(held[0][0, 1], v, rtol=0, atol=tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(setups, tmp_path, dtype):
    folder, reqs, ref = setups["B"]
    steps = traces.mixed(reqs, seed=9)
    out = tmp_path / "out"
    lines = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(traces.peak_tokens(steps))],
                          input=lines, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    vocab = CONFIGS["B"]["vocab_size"]
    pos, rows = {}, {}
    for s in steps:
        keys = []
        for e in s["entries"]:
            p0 = pos.get(e["id"], 0)
            keys += [(e["id"], p0 + w) for w in e["want"]]
            pos[e["id"]] = p0 + len(e["tokens"])
        data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(len(keys), vocab)
        for k, row in zip(keys, data):
            rows[k] = torch.from_numpy(row.copy())
    assert max_diff(rows, ref) < TOL[torch.float32 if dtype == "float32" else torch.bfloat16]
