"""Each CUDA kernel alone against its plain statement (tests/kernel_refs.py), at sizes
other than the engine's: widths and vocabularies that are no power of two, head sizes
in steps of 16, odd head counts and groups, pages of several sizes."""
import math

import pytest
import torch

import kernel_refs as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from wllm_b200.kernels import ops as o
    return o


def tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,H,V", [(1, 64, 100), (37, 2050, 999), (5, 96, 7)])
def test_embed_gather(dtype, n, H, V):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(V, H, generator=g).to(dtype)
    ids = torch.randint(0, V, (n,), generator=g, dtype=torch.int32)
    want = ref.embed_gather(ids, table, 3.25, torch.empty(n, H))
    got = ops().embed_gather(ids.to(DEV), table.to(DEV), 3.25, torch.empty(n, H, device=DEV))
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,H", [(3, 64), (17, 2050), (2, 96), (4, 5000)])
@pytest.mark.parametrize("offset,eps", [(1.0, 1e-6), (0.0, 1e-5)])
def test_rmsnorm_with_and_without_delta_and_rows(dtype, n, H, offset, eps):
    g = torch.Generator().manual_seed(1)
    resid = torch.randn(n, H, generator=g) * 3
    delta = torch.randn(n, H, generator=g).to(dtype)
    w = (torch.randn(H, generator=g) * 0.1).to(dtype)
    # with a delta: the residual is updated in place
    r_ref, out_ref = resid.clone(), torch.empty(n, H, dtype=dtype)
    ref.rmsnorm(r_ref, delta, w, eps, offset, out_ref)
    r_dev, out_dev = resid.to(DEV), torch.empty(n, H, dtype=dtype, device=DEV)
    ops().rmsnorm(r_dev, delta.to(DEV), w.to(DEV), eps, offset, out_dev)
    assert torch.equal(r_dev.cpu(), r_ref)
    torch.testing.assert_close(out_dev.cpu().float(), out_ref.float(), **tol(dtype))
    # without: untouched
    r_dev2, out2 = resid.to(DEV), torch.empty(n, H, dtype=dtype, device=DEV)
    ops().rmsnorm(r_dev2, None, w.to(DEV), eps, offset, out2)
    assert torch.equal(r_dev2.cpu(), resid)
    torch.testing.assert_close(out2.cpu().float(), ref.rmsnorm(resid.clone(), None, w, eps, offset,
                                                              torch.empty(n, H, dtype=dtype)).float(), **tol(dtype))
    # selected rows, delta folded in but not written back
    rows = torch.tensor([n - 1, 0], dtype=torch.int32)
    out3 = torch.empty(2, H, dtype=dtype, device=DEV)
    r_dev3 = resid.to(DEV)
    ops().rmsnorm(r_dev3, delta.to(DEV), w.to(DEV), eps, offset, out3, rows=rows.to(DEV))
    assert torch.equal(r_dev3.cpu(), resid)
    want3 = ref.rmsnorm(resid.clone(), delta, w, eps, offset, torch.empty(2, H, dtype=dtype), rows=rows)
    torch.testing.assert_close(out3.cpu().float(), want3.float(), **tol(dtype))


def test_rmsnorm_32bit_weight_under_bfloat16_output():
    g = torch.Generator().manual_seed(2)
    resid, w = torch.randn(5, 200, generator=g), torch.randn(200, generator=g) * 0.1
    out = torch.empty(5, 200, dtype=torch.bfloat16, device=DEV)
    ops().rmsnorm(resid.to(DEV), None, w.to(DEV), 1e-6, 1.0, out)
    want = ref.rmsnorm(resid.clone(), None, w, 1e-6, 1.0, torch.empty(5, 200, dtype=torch.bfloat16))
    torch.testing.assert_close(out.cpu().float(), want.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pairing", ["half", "interleaved"])
@pytest.mark.parametrize("nq,nkv,hd,rot,ps", [(4, 1, 32, 32, 16), (3, 3, 48, 48, 32), (6, 2, 80, 40, 16), (8, 1, 256, 256, 64)])
def test_rope_kv_write(dtype, nq, nkv, hd, rot, ps, pairing):
    g = torch.Generator().manual_seed(3)
    n, pages = 21, 9
    qkv = torch.randn(n, (nq + 2 * nkv) * hd, generator=g).to(dtype)
    positions = torch.randint(0, 5000, (n,), generator=g, dtype=torch.int32)
    slots = torch.randperm(pages * ps, generator=g)[:n].to(torch.int32)
    slots[4] = -1   # this token writes nothing
    theta = 500.0
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    k_ref = torch.zeros(pages, nkv, ps, hd, dtype=dtype)
    v_ref = torch.zeros_like(k_ref)
    q_ref = torch.zeros(n, nq * hd, dtype=dtype)
    ref.rope_kv_write(qkv, q_ref, positions, slots, inv_freq, k_ref, v_ref, nq, nkv, hd, rot, ps, pairing=pairing)
    q_dev, k_dev, v_dev = (torch.zeros_like(t, device=DEV) for t in (q_ref, k_ref, v_ref))
    ops().rope_kv_write(qkv.to(DEV), q_dev, positions.to(DEV), slots.to(DEV), inv_freq.to(DEV), k_dev, v_dev, nq, nkv, hd,
                        rot, ps, pairing=pairing)
    t = dict(rtol=1e-2, atol=1e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(q_dev.cpu().float(), q_ref.float(), **t)
    torch.testing.assert_close(k_dev.cpu().float(), k_ref.float(), **t)
    assert torch.equal(v_dev.cpu(), v_ref)
    # a layer that reads another layer's cache rotates q and writes no page
    k2 = torch.zeros_like(k_dev)
    ops().rope_kv_write(qkv.to(DEV), q_dev, positions.to(DEV), None, inv_freq.to(DEV), k2, k2, nq, nkv, hd, rot, ps)
    assert float(k2.abs().sum()) == 0.0
    # the row as three float32 partial sums (what a split-K product leaves)
    parts = torch.randn(3, *qkv.shape, generator=g)
    whole = (parts[0] + parts[1]) + parts[2]
    q3, k3, v3 = (torch.zeros_like(t) for t in (q_ref, k_ref, v_ref))
    ref.rope_kv_write(whole, q3, positions, slots, inv_freq, k3, v3, nq, nkv, hd, rot, ps, pairing=pairing)
    q3d, k3d, v3d = (torch.zeros_like(t, device=DEV) for t in (q_ref, k_ref, v_ref))
    ops().rope_kv_write(parts.to(DEV), q3d, positions.to(DEV), slots.to(DEV), inv_freq.to(DEV), k3d, v3d, nq, nkv, hd, rot,
                        ps, in_splits=3, pairing=pairing)
    torch.testing.assert_close(q3d.cpu().float(), q3.float(), **t)
    torch.testing.assert_close(k3d.cpu().float(), k3.float(), **t)
    torch.testing.assert_close(v3d.cpu().float(), v3.float(), **t)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,rot,ps", [(4, 1, 32, 32, 16), (3, 3, 48, 48, 32), (6, 2, 80, 40, 16), (2, 2, 64, 32, 16),
                                              (8, 1, 256, 256, 64)])
def test_rope_kv_write_of_many_tokens_is_the_same_arithmetic(dtype, nq, nkv, hd, rot, ps):
    """From 256 tokens on one CTA walks all heads of a token (16-byte accesses where the sizes allow): the
    reference, and bit for bit what the launch for few tokens writes."""
    g = torch.Generator().manual_seed(5)
    n = 300
    pages = -(-n // ps) + 2
    qkv = torch.randn(n, (nq + 2 * nkv) * hd, generator=g).to(dtype)
    positions = torch.randint(0, 8000, (n,), generator=g, dtype=torch.int32)
    slots = torch.randperm(pages * ps, generator=g)[:n].to(torch.int32)
    slots[7] = -1
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    k_ref = torch.zeros(pages, nkv, ps, hd, dtype=dtype)
    v_ref, q_ref = torch.zeros_like(k_ref), torch.zeros(n, nq * hd, dtype=dtype)
    ref.rope_kv_write(qkv, q_ref, positions, slots, inv_freq, k_ref, v_ref, nq, nkv, hd, rot, ps)
    many = [torch.zeros_like(t, device=DEV) for t in (q_ref, k_ref, v_ref)]
    ops().rope_kv_write(qkv.to(DEV), many[0], positions.to(DEV), slots.to(DEV), inv_freq.to(DEV), many[1], many[2], nq, nkv, hd,
                        rot, ps)
    t = dict(rtol=1e-2, atol=1e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(many[0].cpu().float(), q_ref.float(), **t)
    torch.testing.assert_close(many[1].cpu().float(), k_ref.float(), **t)
    assert torch.equal(many[2].cpu(), v_ref)
    few = [torch.zeros_like(t, device=DEV) for t in (q_ref, k_ref, v_ref)]
    for lo in range(0, n, 100):            # the same rows, a hundred at a time
        ops().rope_kv_write(qkv[lo:lo + 100].to(DEV), few[0][lo:lo + 100], positions[lo:lo + 100].to(DEV),
                            slots[lo:lo + 100].to(DEV), inv_freq.to(DEV), few[1], few[2], nq, nkv, hd, rot, ps)
    for a, b in zip(many, few):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_adds_partial_sums_in_order(dtype):
    g = torch.Generator().manual_seed(8)
    n, H = 6, 2048
    resid, parts = torch.randn(n, H, generator=g), torch.randn(5, n, H, generator=g)
    w = (torch.randn(H, generator=g) * 0.1).to(dtype)
    r_ref, out_ref = resid.clone(), torch.empty(n, H, dtype=dtype)
    ref.rmsnorm(r_ref, parts, w, 1e-6, 1.0, out_ref, delta_splits=5)
    r_dev, out_dev = resid.to(DEV), torch.empty(n, H, dtype=dtype, device=DEV)
    ops().rmsnorm(r_dev, parts.to(DEV), w.to(DEV), 1e-6, 1.0, out_dev, delta_splits=5)
    assert torch.equal(r_dev.cpu(), r_ref)
    torch.testing.assert_close(out_dev.cpu().float(), out_ref.float(), **tol(dtype))


def _paged_case(dtype, nq, nkv, hd, ps, ctx_lens, q_lens, seed, spike=False):
    """Requests with `ctx` tokens in scattered pages; the last `q` of each are this step's queries."""
    g = torch.Generator().manual_seed(seed)
    R = len(ctx_lens)
    pages_each = [-(-c // ps) for c in ctx_lens]
    num_pages = sum(pages_each) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    P = max(pages_each) + 1
    table = torch.full((R, P), -1, dtype=torch.int32)
    k_pages = torch.randn(num_pages, nkv, ps, hd, generator=g).to(dtype)
    v_pages = torch.randn(num_pages, nkv, ps, hd, generator=g).to(dtype)
    it = iter(perm)
    for r in range(R):
        for i in range(pages_each[r]):
            table[r, i] = next(it)
    token_req, positions = [], []
    for r, (c, q) in enumerate(zip(ctx_lens, q_lens)):
        token_req += [r] * q
        positions += list(range(c - q, c))
    n = len(token_req)
    q = (torch.randn(n, nq * hd, generator=g) * (1.0 if not spike else 0.3)).to(dtype)
    if spike:
        # one far key per request gets a score that stands out: a kernel that misses it,
        # or reads it from the wrong page, is far off
        for r, c in enumerate(ctx_lens):
            far = 1 if c > 2 else 0
            page, off = int(table[r, far // ps]), far % ps
            rows = [i for i, t in enumerate(token_req) if t == r]
            k_pages[page, :, off, :] = 0
            k_pages[page, :, off, 0] = 40.0
            for i in rows:
                q[i].view(nq, hd)[:, 0] = 6.0
    return (q, k_pages, v_pages, torch.tensor(token_req, dtype=torch.int32),
            torch.tensor(positions, dtype=torch.int32), table)


ATTN_CASES = [
    # nq nkv hd  ps  ctx_lens            q_lens
    (4, 1, 32, 16, [1, 5, 16, 17, 33, 100], [1, 1, 1, 1, 1, 1]),
    (3, 3, 48, 32, [70, 2, 130], [70, 2, 7]),
    (8, 1, 256, 16, [300, 64, 65], [1, 64, 3]),
    (6, 2, 80, 64, [129, 31], [129, 1]),
    (16, 16, 128, 16, [40], [40]),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ATTN_CASES)
@pytest.mark.parametrize("window", [0, 24])
def test_paged_attention_simt(dtype, case, window):
    nq, nkv, hd, ps, ctx_lens, q_lens = case
    q, kp, vp, treq, pos, table = _paged_case(dtype, nq, nkv, hd, ps, ctx_lens, q_lens, seed=7, spike=(window == 0))
    scale = 1.0 / math.sqrt(hd)
    want = ref.paged_attention(q, torch.empty(q.shape[0], nq * hd, dtype=torch.float64), kp, vp, treq, pos, table,
                               nq, nkv, hd, ps, window, scale, dtype=torch.float64)
    got = torch.empty(q.shape[0], nq * hd, dtype=dtype, device=DEV)
    ops().paged_attention_simt(q.to(DEV), got, kp.to(DEV), vp.to(DEV), treq.to(DEV), pos.to(DEV), table.to(DEV),
                               nq, nkv, hd, ps, window, scale)
    t = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(got.cpu().double(), want, **t)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 300])
def test_paged_attention_simt_split_by_chunks_is_the_walk_bit_for_bit(dtype, window):
    """A warp per (row, chunk of 64 keys) plus the merge kernel gives what one warp per row gives: contexts that
    end inside the first chunk, on a chunk's edge and far behind it, a spike key in the first chunk."""
    nq, nkv, hd, ps = 4, 2, 64, 16
    ctx_lens, q_lens = [1000, 257, 256, 3, 513], [1, 2, 1, 3, 1]
    q, kp, vp, treq, pos, table = _paged_case(dtype, nq, nkv, hd, ps, ctx_lens, q_lens, seed=9, spike=(window == 0))
    scale = 1.0 / math.sqrt(hd)
    args = (kp.to(DEV), vp.to(DEV), treq.to(DEV), pos.to(DEV), table.to(DEV), nq, nkv, hd, ps, window, scale)
    walk = torch.empty(q.shape[0], nq * hd, dtype=dtype, device=DEV)
    ops().paged_attention_simt(q.to(DEV), walk, *args)
    want = ref.paged_attention(q, torch.empty(q.shape[0], nq * hd, dtype=torch.float64), kp, vp, treq, pos, table,
                               nq, nkv, hd, ps, window, scale, dtype=torch.float64)
    t = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(walk.cpu().double(), want, **t)
    chunks = ops().simt_chunks(max(ctx_lens), window)
    assert chunks == (16 if window == 0 else 6)
    for bound in (chunks, chunks + 2):
        scratch = torch.full((q.shape[0] * nq * bound * (hd + 2),), float("nan"), device=DEV)
        split = torch.full_like(walk, float("nan"))
        ops().paged_attention_simt(q.to(DEV), split, *args, scratch=scratch, max_chunks=bound)
        assert torch.equal(split, walk)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 70])
@pytest.mark.parametrize("case", [
    (4, 2, 64, 16, [300, 257, 64, 3, 130], [300, 2, 33, 3, 1]),      # whole prompts, portions behind a prefix, one token
    (8, 1, 256, 64, [200, 700], [200, 37]),                          # eight heads of a group share a tile's rows
    (3, 3, 48, 32, [100, 65], [31, 65]),
    (16, 16, 128, 16, [90], [90]),
])
def test_paged_attention_simt_tiled_is_the_walk_bit_for_bit(dtype, window, case):
    """32 rows of a request against every tile of keys brought into shared memory once: the same numbers as a warp
    per row, to the last bit, and the float64 statement within tolerance; rows that end inside a tile, inside a
    chunk and on a chunk's edge, a window that starts inside a tile."""
    nq, nkv, hd, ps, ctx_lens, q_lens = case
    q, kp, vp, treq, pos, table = _paged_case(dtype, nq, nkv, hd, ps, ctx_lens, q_lens, seed=13, spike=(window == 0))
    table = table.clamp(min=0)
    scale = 1.0 / math.sqrt(hd)
    starts = [sum(q_lens[:r]) for r in range(len(q_lens))]
    meta = [torch.tensor(x, dtype=torch.int32, device=DEV) for x in (starts, q_lens, ctx_lens)]
    qd, kd, vd, td = q.to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV)
    walk = torch.empty(q.shape[0], nq * hd, dtype=dtype, device=DEV)
    ops().paged_attention_simt(qd, walk, kd, vd, treq.to(DEV), pos.to(DEV), td, nq, nkv, hd, ps, window, scale)
    tiled = torch.full_like(walk, float("nan"))
    ops().paged_attention_simt_tiled(qd, tiled, kd, vd, *meta, td, max(q_lens), nq, nkv, hd, ps, window, scale)
    assert torch.equal(tiled, walk)
    want = ref.paged_attention(q, torch.empty(q.shape[0], nq * hd, dtype=torch.float64), kp, vp, treq, pos, table,
                               nq, nkv, hd, ps, window, scale, dtype=torch.float64)
    t = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(tiled.cpu().double(), want, **t)


def test_paged_attention_refuses_unsupported_head_size():
    from wllm_b200.kernels import KernelError
    q = torch.zeros(1, 40, device=DEV)
    kp = torch.zeros(1, 1, 16, 40, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="size not supported"):
        ops().paged_attention_simt(q, torch.empty_like(q), kp, kp, z, z, z.view(1, 1), 1, 1, 40, 16, 0, 1.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
@pytest.mark.parametrize("n,I", [(1, 256), (19, 384), (3, 1001)])
def test_gated_act(dtype, act, n, I):
    g = torch.Generator().manual_seed(4)
    gu = (torch.randn(n, 2 * I, generator=g) * 2).to(dtype)
    want = ref.gated_act(gu, torch.empty(n, I, dtype=dtype), act)
    got = ops().gated_act(gu.to(DEV), torch.empty(n, I, dtype=dtype, device=DEV), act)
    torch.testing.assert_close(got.cpu().float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("M,N,K", [(1, 512, 64), (33, 1000, 96), (130, 257, 144), (7, 129, 50), (300, 300, 1027),
                                   (12, 3080, 520), (20, 100, 136), (32, 48, 2048), (64, 250, 1000), (5, 7, 4)])
def test_gemm_f32_is_true_32bit_and_row_invariant(M, N, K):
    g = torch.Generator().manual_seed(5)
    a, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    want = (a.double() @ w.double().t())
    got = ops().gemm_f32(a.to(DEV), w.to(DEV)).cpu()
    # 32-bit accumulation error grows with sqrt(K); a reduced-precision mode would be ~1e-3 off
    assert float((got.double() - want).abs().max()) < 2e-6 * math.sqrt(K) * 10
    # a row of the result does not depend on the other rows of the batch
    alone = ops().gemm_f32(a[M // 2: M // 2 + 1].to(DEV), w.to(DEV)).cpu()
    assert torch.equal(alone[0], got[M // 2])


def _mma_inputs(case, seed, spike=True):
    nq, nkv, hd, ps, ctx_lens, q_lens = case
    q, kp, vp, treq, pos, table = _paged_case(torch.bfloat16, nq, nkv, hd, ps, ctx_lens, q_lens, seed, spike)
    table = table.clamp(min=0)
    starts, s = [], 0
    for n in q_lens:
        starts.append(s)
        s += n
    meta = [torch.tensor(x, dtype=torch.int32, device=DEV) for x in (starts, q_lens, ctx_lens)]
    return q, kp, vp, treq, pos, table, meta


MMA_CASES = ATTN_CASES + [
    (8, 1, 256, 64, [1000, 1, 700, 64], [1, 1, 1, 1]),
    (8, 1, 256, 16, [1030], [1030]),
    (16, 16, 256, 32, [200, 77], [5, 77]),
    (4, 2, 96, 16, [500, 333, 2], [1, 300, 2]),
    (4, 2, 128, 32, [700, 90], [300, 90]),          # head size 128, tiles of 256 rows on pairs of CTAs
    (6, 2, 64, 16, [700, 65, 1, 300], [1, 1, 1, 1]),  # head size 64: the smallest that the TMA kernels take
    (6, 2, 64, 32, [300, 130], [140, 2]),
]


@pytest.mark.parametrize("case", MMA_CASES)
@pytest.mark.parametrize("window", [0, 24])
@pytest.mark.parametrize("split_keys", [64, 256])
def test_attention_mma_decode_and_prefill_cover_a_mixed_batch(case, window, split_keys):
    """split_keys 64 also lets two prefill CTAs share every tile that walks more than two key tiles."""
    nq, nkv, hd, ps, ctx_lens, q_lens = case
    q, kp, vp, treq, pos, table, (starts, qlens, ctxs) = _mma_inputs(case, seed=11, spike=(window == 0))
    scale = 1.0 / math.sqrt(hd)
    want = ref.paged_attention(q, torch.empty(q.shape[0], nq * hd, dtype=torch.float64), kp, vp, treq, pos, table,
                               nq, nkv, hd, ps, window, scale, dtype=torch.float64)
    got = torch.full((q.shape[0], nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    o = ops()
    R = len(q_lens)
    max_splits = -(-max(ctx_lens) // split_keys)
    scratch = torch.full((o.attention_mma_scratch_floats(R, nq, hd, max_splits),), float("nan"), device=DEV)
    qd, kd, vd, td = q.to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV)
    decode = any(n == 1 for n in q_lens)
    if decode:
        o.attention_mma_decode(qd, got, kd, vd, starts, qlens, ctxs, td, nq, nkv, hd, ps, window, scale, split_keys,
                               max_splits, scratch)
    if any(n > 1 for n in q_lens) or not decode:
        share = 2 if (hd % 64 == 0 and split_keys == 64) else 0
        halves = torch.full((o.attention_prefill_halves_floats(R, max(q_lens), nq, nkv, hd),), float("nan"), device=DEV) \
            if share else None
        o.attention_mma_prefill(qd, got, kd, vd, starts, qlens, ctxs, td, max(q_lens), nq, nkv, hd, ps, window, scale,
                                skip_single=decode, split_above=share, halves=halves)
        if share:       # whichever of the two CTAs merges, the result is the same
            again = torch.full_like(got, float("nan"))
            o.attention_mma_prefill(qd, again, kd, vd, starts, qlens, ctxs, td, max(q_lens), nq, nkv, hd, ps, window,
                                    scale, skip_single=decode, split_above=share, halves=halves)
            rows = torch.cat([torch.arange(s, s + n) for s, n in zip(starts.tolist(), q_lens) if n > 1 or not decode])
            assert torch.equal(again[rows.to(DEV)], got[rows.to(DEV)])
    torch.testing.assert_close(got.cpu().double(), want, rtol=2e-2, atol=2e-2)


def test_attention_mma_prefill_alone_serves_single_tokens_too():
    case = (8, 1, 256, 64, [300, 1, 64], [1, 1, 1])
    nq, nkv, hd, ps, ctx_lens, q_lens = case
    q, kp, vp, treq, pos, table, (starts, qlens, ctxs) = _mma_inputs(case, seed=12)
    scale = 1.0 / math.sqrt(hd)
    want = ref.paged_attention(q, torch.empty(3, nq * hd, dtype=torch.float64), kp, vp, treq, pos, table, nq, nkv, hd,
                               ps, 0, scale, dtype=torch.float64)
    got = torch.full((3, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops().attention_mma_prefill(q.to(DEV), got, kp.to(DEV), vp.to(DEV), starts, qlens, ctxs, table.to(DEV), 1, nq, nkv,
                                hd, ps, 0, scale, skip_single=False)
    torch.testing.assert_close(got.cpu().double(), want, rtol=2e-2, atol=2e-2)
