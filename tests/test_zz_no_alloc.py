"""The allocation-free decode attention entry point (csrc/attention_decode_static.h), called
through its exported C symbol the way an embedding host would, against the engine's own
entry point, which takes its scratch from the caller.

Some hosts may not allocate device memory at all (their memory is owned elsewhere, or they
run where cudaMalloc is off limits); for them the partial results of the key splits live in
a fixed array inside the library.  The two entry points run the same kernels, so their
outputs must agree to the last bit; both are also held against the float64 statement of
paged attention in tests/kernel_refs.py, within the tolerance of the other kernel tests (a
fault in what the two share would otherwise pass).  Two calls in a row share the array:
the second must not see the first.  A window, and a context beyond the caller's plan of
splits, go through the fixed array as well."""
import ctypes
import math
from ctypes import c_float, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HD = 64


def _case(seed, nq, nkv, ps, ctx_lens):
    g = torch.Generator().manual_seed(seed)
    R = len(ctx_lens)
    pages_each = [-(-c // ps) for c in ctx_lens]
    num_pages = sum(pages_each) + 2
    perm = iter(torch.randperm(num_pages, generator=g).tolist())
    table = torch.zeros((R, max(pages_each)), dtype=torch.int32)
    for r in range(R):
        for i in range(pages_each[r]):
            table[r, i] = next(perm)
    k = torch.randn(num_pages, nkv, ps, HD, generator=g).to(torch.bfloat16)
    v = torch.randn(num_pages, nkv, ps, HD, generator=g).to(torch.bfloat16)
    q = torch.randn(R, nq * HD, generator=g).to(torch.bfloat16)
    meta = [torch.tensor(x, dtype=torch.int32, device=DEV) for x in (list(range(R)), [1] * R, ctx_lens)]
    return q.to(DEV), k.to(DEV), v.to(DEV), table.to(DEV), meta


def _call_static(lib, q, out, k, v, table, meta, nq, nkv, ps, scale, split_keys, max_splits, window=0):
    starts, qlens, ctxs = meta
    p = lambda t: c_void_p(t.data_ptr())   # noqa: E731
    status = torch.zeros(1, dtype=torch.int32, device=DEV)     # stays 0 unless a bounded wait in the kernel ran out
    rc = lib.wllm_attention_mma_decode_static(
        p(q), q.stride(0), p(out), out.stride(0), p(k), p(v), ctypes.c_longlong(k.shape[0]), p(starts), p(qlens), p(ctxs),
        p(table), table.shape[1], qlens.shape[0], nq, nkv, ps, window, c_float(scale), split_keys, max_splits, p(status),
        c_void_p(torch.cuda.current_stream().cuda_stream))
    assert int(status.item()) == 0
    return rc


def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row():
    from wllm_b200.kernels import ops
    from wllm_b200.kernels.build import load_family
    lib = load_family("attention_decode_static", {"HEAD_DIM": HD})
    assert isinstance(lib, ctypes.CDLL)
    lib.wllm_attention_mma_decode_static_needs.restype = ctypes.c_longlong
    import kernel_refs as ref
    nq, nkv, ps, scale = 6, 2, 16, 1.0 / math.sqrt(HD)
    # (seed, contexts, keys per split, splits, window); the last plan covers 256 keys of a 700-key context
    for seed, ctx_lens, split_keys, max_splits, window in ((1, [700, 65, 1, 300], 128, 6, 0), (2, [33, 512, 129], 64, 8, 0),
                                                          (3, [700, 40, 200], 64, 11, 50), (4, [700, 65], 64, 4, 0)):
        q, k, v, table, meta = _case(seed, nq, nkv, ps, ctx_lens)
        R = len(ctx_lens)
        want = torch.full((R, nq * HD), float("nan"), dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(ops.attention_mma_scratch_floats(R, nq, HD, max_splits), device=DEV)
        ops.attention_mma_decode(q, want, k, v, *meta, table, nq, nkv, HD, ps, window, scale, split_keys, max_splits, scratch)
        assert lib.wllm_attention_mma_decode_static_needs(R, nq, max_splits) == scratch.numel()
        got = torch.full_like(want, float("nan"))
        assert _call_static(lib, q, got, k, v, table, meta, nq, nkv, ps, scale, split_keys, max_splits, window) == 0
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(got, want)
        positions = torch.tensor([c - 1 for c in ctx_lens], dtype=torch.int32)
        exact = ref.paged_attention(q.cpu(), torch.empty(R, nq * HD, dtype=torch.float64), k.cpu(), v.cpu(),
                                    torch.arange(R, dtype=torch.int32), positions, table.cpu(), nq, nkv, HD, ps, window,
                                    scale, dtype=torch.float64)
        torch.testing.assert_close(got.cpu().double(), exact, rtol=2e-2, atol=2e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from wllm_b200.kernels.build import load_family
    lib = load_family("attention_decode_static", {"HEAD_DIM": HD})
    q, k, v, table, meta = _case(3, 8, 8, 16, [64] * 64)
    out = torch.zeros_like(q)
    # 64 requests x 8 heads x 64 splits x 66 floats is above the array's 2^20 floats: nothing runs
    assert _call_static(lib, q, out, k, v, table, meta, 8, 8, 16, 1.0, 64, 64) == 4
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0
