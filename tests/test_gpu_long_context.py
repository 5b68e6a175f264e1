"""The tensor-core attention kernels and the engine at the context lengths that the benchmark and the
continuous-batching workload run: 4,096 to 8,192 cached keys under 1, 8 and 64 requests, portions of
2,048 tokens on 6,144 cached keys, a 5,000-token prompt.  Operands are made on the device; the float64
statement of tests/kernel_refs.py is evaluated there too, for a handful of rows, so that the cost stays small.
The split plans are the ones the step context would choose (`ops.decode_split_plan`), not the test's own."""
import math
import os
import subprocess
import sys

import pytest
import torch

import kernel_refs as ref
import plain_gemma as plain
import traces

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HD, PS = 256, 64


def paged_case(nq, nkv, ctx_lens, q_lens, seed, spike):
    """Requests with `ctx` tokens in scattered pages of 64, the last `q` of each being this step's queries.
    `spike`: key 1 of every request gets a score that stands out far behind thousands of others, so a kernel
    that drops it or reads another page's row is far off; without it every key carries weight."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    R = len(ctx_lens)
    pages_each = [-(-c // PS) for c in ctx_lens]
    num_pages = sum(pages_each) + 3
    perm = torch.randperm(num_pages, generator=g, device=DEV).to(torch.int32)
    # (entries of the table behind a request's pages name a page that holds numbers, as a real table's do)
    table = torch.full((R, max(pages_each) + 1), int(perm[0]), dtype=torch.int32, device=DEV)
    at = 0
    for r, n in enumerate(pages_each):
        table[r, :n] = perm[at:at + n]
        at += n
    k_pages = torch.randn(num_pages, nkv, PS, HD, generator=g, device=DEV).to(torch.bfloat16)
    v_pages = torch.randn(num_pages, nkv, PS, HD, generator=g, device=DEV).to(torch.bfloat16)
    token_req = torch.cat([torch.full((q,), r, dtype=torch.int32) for r, q in enumerate(q_lens)]).to(DEV)
    positions = torch.cat([torch.arange(c - q, c, dtype=torch.int32) for c, q in zip(ctx_lens, q_lens)]).to(DEV)
    q = (torch.randn(sum(q_lens), nq * HD, generator=g, device=DEV) * (0.3 if spike else 1.0)).to(torch.bfloat16)
    if spike:
        for r, c in enumerate(ctx_lens):
            far = 1 if c > 2 else 0
            k_pages[int(table[r, 0]), :, far, :] = 0
            k_pages[int(table[r, 0]), :, far, 0] = 40.0
        q.view(-1, nq, HD)[:, :, 0] = 6.0
    # what lies behind a request's last key in its last page, and the pages nobody holds, is no number at all
    for r, c in enumerate(ctx_lens):
        if c % PS:
            last = int(table[r, (c - 1) // PS])
            k_pages[last, :, c % PS:, :] = float("nan")
            v_pages[last, :, c % PS:, :] = float("nan")
    k_pages[perm[at:].long()] = float("nan")
    v_pages[perm[at:].long()] = float("nan")
    starts = [sum(q_lens[:r]) for r in range(R)]
    meta = [torch.tensor(x, dtype=torch.int32, device=DEV) for x in (starts, q_lens, ctx_lens)]
    return q, k_pages, v_pages, token_req, positions, table, meta


def check_rows(got, rows, q, k_pages, v_pages, token_req, positions, table, nq, nkv, what):
    rows = torch.tensor(sorted(r for r in set(rows) if 0 <= r < q.shape[0]), device=DEV)
    want = ref.paged_attention(q[rows], torch.empty(len(rows), nq * HD, dtype=torch.float64, device=DEV), k_pages, v_pages,
                               token_req[rows], positions[rows], table, nq, nkv, HD, PS, 0, 1.0 / math.sqrt(HD),
                               dtype=torch.float64)
    assert not torch.isnan(got.float()).any(), f"{what}: rows that no CTA wrote"
    worst = float((got[rows].double() - want).abs().max())
    assert worst < 2e-2, f"{what}: largest difference {worst:.3e} (values of order {float(want.abs().max()):.2f})"


@pytest.mark.parametrize("heads", [(8, 1), (16, 16)], ids=["mqa8", "mha16"])
@pytest.mark.parametrize("requests", [1, 8, 64])
@pytest.mark.parametrize("context", [4096, 8165, 8192])
def test_decode_attention_at_the_benchmark_contexts(context, requests, heads):
    """16 and 64 requests at 8,192 keys is the case in which the first warp-specialised decode kernel failed."""
    from wllm_b200.kernels import ops
    nq, nkv = heads
    ctx_lens = [context] * requests
    if requests > 1:
        ctx_lens[1], ctx_lens[-1] = 777, context - 1
    case = paged_case(nq, nkv, ctx_lens, [1] * requests, seed=context + requests, spike=requests != 8)
    q, k_pages, v_pages, token_req, positions, table, (starts, qlens, ctxs) = case
    split_keys, max_splits = ops.decode_split_plan(requests * nkv, -(-max(ctx_lens) // 512) * 512, 32)
    scratch = torch.full((ops.attention_mma_scratch_floats(requests, nq, HD, max_splits),), float("nan"), device=DEV)
    got = torch.full((requests, nq * HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_mma_decode(q, got, k_pages, v_pages, starts, qlens, ctxs, table, nq, nkv, HD, PS, 0, 1.0 / math.sqrt(HD),
                             split_keys, max_splits, scratch)
    assert ops.tc_gemm_status(DEV) == 0
    check_rows(got, [0, min(1, requests - 1), requests // 2, requests - 1], *case[:6], nq, nkv,
               f"{requests} requests x {context} keys, plan {split_keys} x {max_splits}")


PREFILL_CASES = {
    # nq nkv cached new        which kernel serves it
    "pairs_2048_on_6144": (8, 1, 6144, 2048),     # pairs of CTAs on 256-row tiles (every portion of a long prompt)
    "pairs_mha_300_on_6000": (16, 16, 6000, 300),
    "single_100_on_6000": (16, 16, 6000, 100),    # one tile of rows: one CTA a tile, 64-key tiles
    "pairs_2048_from_0": (8, 1, 0, 2048),
}


@pytest.mark.parametrize("name", list(PREFILL_CASES))
def test_prefill_attention_over_a_long_cached_prefix(name):
    """With WLLM_ATTENTION_PAIR=0 in the environment the same cases run on the one-CTA-a-tile kernel."""
    from wllm_b200.kernels import ops
    nq, nkv, cached, new = PREFILL_CASES[name]
    case = paged_case(nq, nkv, [cached + new, 700], [new, 2], seed=cached + new, spike=(nkv == 1))
    q, k_pages, v_pages, token_req, positions, table, (starts, qlens, ctxs) = case
    got = torch.full((new + 2, nq * HD), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_mma_prefill(q, got, k_pages, v_pages, starts, qlens, ctxs, table, new, nq, nkv, HD, PS, 0,
                              1.0 / math.sqrt(HD), skip_single=False)
    assert ops.tc_gemm_status(DEV) == 0
    check_rows(got, [0, 1, 31, 32, 127, 128, new // 2, new - 1, new, new + 1], *case[:6], nq, nkv, name)


def test_prefill_attention_over_a_long_prefix_on_the_one_cta_kernel():
    """The same long-prefix cases in a process of their own in which pairs of CTAs are switched off (the
    switch is read once a process), so that `prefill_tc_kernel` walks the 6,000 cached keys."""
    env = dict(os.environ, WLLM_ATTENTION_PAIR="0")
    proc = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-m", "gpu", "-x", "-q", "-k",
                           "test_prefill_attention_over_a_long_cached_prefix"], env=env, capture_output=True, text=True,
                          timeout=900)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-1000:]
    assert "4 passed" in proc.stdout


# -- the engine at Gemma-2B's layer widths over a 5,000-token prompt ---------------------------------------

WIDTHS_2B = dict(hidden_size=2048, num_attention_heads=8, num_key_value_heads=1, head_dim=256, intermediate_size=16384)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_engine_over_a_5000_token_prompt_whole_in_portions_and_token_by_token(dtype):
    """Two layers at Gemma-2B's widths, a vocabulary of 4,096 (so that every position's logits can be kept), one
    5,000-token prompt: whole, in portions of 512, and with its last 32 tokens one by one (decode attention
    over 5,000 keys, the split plan of a lone request).  Against the plain implementation on the same weights
    (on the device, float32); in 32-bit the three ways also agree bit for bit."""
    from test_gpu_fp32_equality import plain_weights
    from wllm_b200.config import EngineConfig, GemmaConfig
    from wllm_b200.engine import build_model, build_runner
    raw = dict(architectures=["GemmaForCausalLM"], model_type="gemma", num_hidden_layers=2, vocab_size=4096,
               max_position_embeddings=8192, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, **WIDTHS_2B)
    torch.backends.cuda.matmul.allow_tf32 = False
    ec = EngineConfig(dtype=dtype, block_size=64, max_num_seqs=4)
    model = build_model(None, dtype, ec.device, config=GemmaConfig.from_dict(raw), random_seed=12)
    g = torch.Generator().manual_seed(13)
    reqs = {"long": torch.randint(0, 4096, (5000,), generator=g).tolist()}
    want = plain.forward(reqs["long"], {k: v.float() for k, v in plain_weights(model, raw).items()}, raw)
    scale = float(want.abs().max())
    first = None
    for cut, steps in (("whole", traces.whole(reqs)), ("portions", traces.portions(reqs, sizes=(512,))),
                       ("tail", traces.tail_singly(reqs, tail=32))):
        runner = build_runner(model, ec, num_pages=-(-5000 // 64) + 1, poison_pages=True)
        rows = traces.run_in_process(runner, steps)
        got = torch.stack([rows[("long", p)] for p in range(5000)]).to(DEV)
        worst = float((got.double() - want.double()).abs().max())
        bound = 2e-4 if dtype == torch.float32 else 0.004 * max(1.0, scale)
        assert worst < bound, f"{cut}: largest difference {worst:.3e} on logits of up to {scale:.2f} (bound {bound:.1e})"
        if dtype == torch.float32:
            if first is None:
                first = got
            else:
                bad = (first != got).any(dim=1).nonzero()
                assert bad.numel() == 0, f"{cut}: first differing position {int(bad[0])}"
