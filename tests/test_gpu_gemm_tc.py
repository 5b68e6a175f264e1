"""The tcgen05 / tensor-memory GEMM against a float64 product of the same bfloat16 operands,
at sizes that are no multiples of its tiles, with every epilogue."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SIZES = [(128, 256, 64), (128, 256, 256), (256, 512, 128), (300, 1000, 96), (1, 512, 64), (77, 130, 144),
         (2048, 2560, 2048), (513, 2048, 4096)]


def operands(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.5).to(torch.bfloat16)
    return a, w


@pytest.mark.parametrize("M,N,K", SIZES)
@pytest.mark.parametrize("epilogue", ["bf16", "f32"])
def test_plain_product(M, N, K, epilogue):
    from wllm_b200.kernels import ops
    a, w = operands(M, N, K, seed=M + N + K)
    want = a.double() @ w.double().T
    got = ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), epilogue=epilogue)
    torch.cuda.synchronize()
    assert ops.tc_gemm_status(DEV) == 0
    if epilogue == "f32":
        assert got.dtype == torch.float32
        torch.testing.assert_close(got.cpu().double(), want, rtol=1e-4, atol=1e-3 * math.sqrt(K))
    else:
        torch.testing.assert_close(got.cpu().double(), want, rtol=1e-2, atol=2e-2 * math.sqrt(K))


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (200, 384, 96), (64, 1000, 64), (2048, 16384, 2048)])
@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
def test_gated_epilogue(M, I, K, act):
    from wllm_b200.kernels import ops
    a, w = operands(M, 2 * I, K, seed=I)
    a, w = a * 0.3, w * 0.3
    a, w = a.to(torch.bfloat16), w.to(torch.bfloat16)
    gate, up = a.double() @ w[:I].double().T, a.double() @ w[I:].double().T
    f = torch.nn.functional
    want = (f.gelu(gate, approximate="tanh") if act == "gelu_tanh" else f.silu(gate)) * up
    got = ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), epilogue=act)
    torch.cuda.synchronize()
    assert ops.tc_gemm_status(DEV) == 0 and got.shape == (M, I)
    torch.testing.assert_close(got.cpu().double(), want, rtol=2e-2, atol=2e-2 * math.sqrt(K))


def test_rows_do_not_depend_on_the_batch_and_strided_operands_work():
    from wllm_b200.kernels import ops
    a, w = operands(300, 520, 256, seed=9)
    ad, wd = a.to(DEV), w.to(DEV)
    full = ops.gemm_bf16_tc(ad, wd)
    part = ops.gemm_bf16_tc(ad[131:140], wd)
    assert torch.equal(full[131:140], part)
    wide = torch.zeros(300, 512, dtype=torch.bfloat16, device=DEV)
    wide[:, :256] = ad
    assert torch.equal(ops.gemm_bf16_tc(wide[:, :256], wd), full)
    out = torch.zeros(300, 1024, dtype=torch.bfloat16, device=DEV)
    ops.gemm_bf16_tc(ad, wd, out=out[:, 8:528])
    assert torch.equal(out[:, 8:528], full) and float(out[:, 528:].abs().sum()) == 0


def test_refuses_what_it_cannot_take():
    from wllm_b200.kernels import KernelError, ops
    a = torch.zeros(8, 20, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="steps of 8"):
        ops.gemm_bf16_tc(a, torch.zeros(16, 20, dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("M,N,K", [(8, 2048, 2048), (8, 2560, 2048), (64, 2048, 16384), (1, 512, 200), (33, 300, 1024),
                                   (100, 2560, 2048), (128, 2048, 16384), (256, 2048, 16384), (300, 2560, 2048), (512, 2048, 2048),
                                   (700, 3072, 24576)])
def test_split_k_partial_sums(M, N, K):
    """Up to 128 rows on single CTAs, above on pairs: the parts of K that the plan gives, slab by slab."""
    from wllm_b200.kernels import ops
    a, w = operands(M, N, K, seed=K + M)
    want = a.double() @ w.double().T
    half, parts = ops.product_plan(M, N, K)
    assert parts >= 1 and (K <= 64 or parts > 1)
    out = torch.full((parts, M, N), float("nan"), device=DEV)
    if parts > 1:
        ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), out=out, epilogue="f32", k_splits=parts, half_rows=half)
    else:
        ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), out=out[0], epilogue="f32")
    torch.cuda.synchronize()
    assert ops.tc_gemm_status(DEV) == 0
    total = out.cpu().double().sum(0)
    torch.testing.assert_close(total, want, rtol=1e-4, atol=1e-3 * math.sqrt(K))
    again = torch.empty_like(out)
    ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), out=again if parts > 1 else again[0], epilogue="f32", k_splits=parts, half_rows=half)
    assert torch.equal(again, out)        # part s is the same sum whoever computes it


@pytest.mark.parametrize("M,half", [(8, 48), (8, 64), (8, 112), (40, 32), (64, 80), (100, 16), (128, 96), (31, 128),
                                    (300, 80), (257, 16), (512, 112), (260, 64)])     # from 129 rows on: pairs of CTAs
@pytest.mark.parametrize("epilogue", ["f32", "bf16", "gelu_tanh"])
def test_every_tile_shape_of_products_of_few_rows(M, half, epilogue):
    """The W tile of a stage is two halves of `half` rows (one half in each CTA of a pair): every multiple of 16
    the row count allows, at an N and K that are multiples of nothing."""
    from wllm_b200.kernels import ops
    I, K = 300, 200
    a, w = operands(M, 2 * I, K, seed=half + M)
    want = a.double() @ w.double().T
    if epilogue == "gelu_tanh":
        a, w = (a * 0.3).to(torch.bfloat16), (w * 0.3).to(torch.bfloat16)
        want = torch.nn.functional.gelu(a.double() @ w[:I].double().T, approximate="tanh") * (a.double() @ w[I:].double().T)
    got = ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), epilogue=epilogue, half_rows=half)
    torch.cuda.synchronize()
    assert ops.tc_gemm_status(DEV) == 0 and got.shape == want.shape
    if epilogue == "f32":
        torch.testing.assert_close(got.cpu().double(), want, rtol=1e-4, atol=1e-3 * math.sqrt(K))
        assert torch.equal(got, ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), epilogue="f32", half_rows=128 if M > 32 else 48))
    else:
        torch.testing.assert_close(got.cpu().double(), want, rtol=2e-2, atol=2e-2 * math.sqrt(K))


@pytest.mark.parametrize("M,N,K,half", [(300, 1000, 200, 120), (300, 1000, 200, 72), (257, 600, 136, 144), (700, 1300, 200, 144),
                                        (512, 1100, 328, 192), (300, 1030, 200, 256), (2048, 2560, 2048, 144),
                                        (2048, 2048, 1024, 120), (3000, 5000, 256, 144)])
@pytest.mark.parametrize("epilogue", ["f32", "bf16"])
def test_tile_widths_of_pairs(M, N, K, half, epilogue):
    """On pairs of CTAs a half may be any multiple of 8, and halves of 144 to 256 rows make wide tiles (one
    accumulator, two products a step, each CTA's half in two boxes); the last case runs several rounds of
    wide tiles, where the products of a tile wait for the drain of the tile before."""
    from wllm_b200.kernels import ops
    a, w = operands(M, N, K, seed=half + M)
    want = a.double() @ w.double().T
    got = ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), epilogue=epilogue, half_rows=half)
    torch.cuda.synchronize()
    assert ops.tc_gemm_status(DEV) == 0 and got.shape == want.shape
    if epilogue == "f32":
        torch.testing.assert_close(got.cpu().double(), want, rtol=1e-4, atol=1e-3 * math.sqrt(K))
        assert torch.equal(got, ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), epilogue="f32", half_rows=128))
    else:
        torch.testing.assert_close(got.cpu().double(), want, rtol=1e-2, atol=2e-2 * math.sqrt(K))


@pytest.mark.parametrize("M,N,K", [(2048, 3072, 4096), (2048, 12288, 3072), (2100, 3072, 24576), (2048, 2560, 2048), (4096, 2560, 2048)])
def test_the_planned_widths_at_the_shapes_of_gemma_7b_and_2b(M, N, K):
    """The widths that the plan picks for prompts at the real shapes (halves of 144 to 240 rows), against a float64
    product of the same operands formed on the device, and bit-equal to tiles of 256 columns."""
    from wllm_b200.kernels import ops
    g = torch.Generator(device=DEV).manual_seed(M + N)
    a = (torch.randn(M, K, generator=g, device=DEV) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device=DEV) * 0.5).to(torch.bfloat16)
    half, _ = ops.tile_plan(M, N, K, False, False)
    got = ops.gemm_bf16_tc(a, w, epilogue="f32")
    torch.cuda.synchronize()
    assert ops.tc_gemm_status(DEV) == 0
    assert torch.equal(got, ops.gemm_bf16_tc(a, w, epilogue="f32", half_rows=128)), half
    rows = torch.tensor([0, 1, 127, 128, 255, 256, M // 2, M - 1], device=DEV)
    want = a[rows].double() @ w.double().T
    torch.testing.assert_close(got[rows].double(), want, rtol=1e-4, atol=1e-3 * math.sqrt(K))


def test_wide_tiles_are_refused_where_they_do_not_exist():
    from wllm_b200.kernels import KernelError, ops
    a, w = operands(300, 1024, 64, seed=1)
    with pytest.raises(KernelError):
        ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), half_rows=144, epilogue="gelu_tanh")     # the gate and up halves are the tile
    with pytest.raises(KernelError):
        ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), half_rows=152)                           # steps of 16 above 128
    with pytest.raises(KernelError):
        ops.gemm_bf16_tc(a[:100].to(DEV), w.to(DEV), half_rows=144)                      # one CTA a tile: two accumulators of 256
    with pytest.raises(KernelError):
        ops.gemm_bf16_tc(a[:100].to(DEV), w.to(DEV), half_rows=120)


def test_a_wide_tile_as_the_first_product_of_a_process():
    """How many pairs the device holds is asked of the plain form of the kernel; a process whose first product is
    a wide one must get the same answer."""
    import subprocess
    import sys
    code = ("import torch; from wllm_b200.kernels import ops; "
            "a = torch.ones(300, 64, dtype=torch.bfloat16, device='cuda:0'); "
            "w = torch.ones(1000, 64, dtype=torch.bfloat16, device='cuda:0'); "
            "c = ops.gemm_bf16_tc(a, w, epilogue='f32', half_rows=144); torch.cuda.synchronize(); "
            "assert float(c.min()) == 64.0 == float(c.max()), c; print('ok', ops.resident_pairs())")
    done = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert done.returncode == 0 and done.stdout.startswith("ok"), done.stderr[-2000:]


def test_the_plan_for_many_rows_saves_rounds():
    from wllm_b200.kernels import ops
    pairs = ops.resident_pairs()
    for M, N, K in [(2048, 2560, 2048), (2048, 2048, 16384), (2048, 12288, 3072), (2048, 3072, 24576), (2100, 3072, 24576),
                    (300, 2560, 2048), (129, 100, 64)]:
        half, parts = ops.tile_plan(M, N, K, False, False)
        assert parts == 1 and half % 16 == 0 and 64 <= half <= 256
        rounds = lambda h: -(-(-(-M // 256) * -(-N // (2 * h))) // pairs)
        assert rounds(half) * half <= rounds(128) * 128         # never more columns walked than with tiles of 256
    if pairs == 74:
        assert ops.tile_plan(2048, 2560, 2048, False, False) == (144, 1)      # 72 tiles instead of 80
        assert ops.tile_plan(2048, 2048, 16384, False, False) == (128, 1)     # 64 tiles: nothing to save
        assert ops.tile_plan(2048, 32768, 2048, True, False) == (128, 1)      # the gate keeps its halves


def test_a_tile_too_small_for_the_row_count_is_refused():
    from wllm_b200.kernels import KernelError, ops
    a, w = operands(8, 256, 64, seed=1)
    with pytest.raises(KernelError):
        ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), half_rows=32)      # 32 rows of A + 2 x 32 of W < the 128 rows read at A
    with pytest.raises(KernelError):
        ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), half_rows=40)


def test_tile_plan_fills_the_sms():
    from wllm_b200.kernels import ops
    for M, N, K, gated, split in [(8, 2560, 2048, False, True), (8, 2048, 16384, False, True), (8, 32768, 2048, True, False),
                                  (64, 2048, 2048, False, True), (1, 512, 200, False, True), (33, 300, 1024, False, True)]:
        half, parts = ops.tile_plan(M, N, K, gated, split)
        assert half % 16 == 0 and 16 <= half <= 128 and 1 <= parts <= 16
        assert half >= (48 if M <= 32 else 32 if M <= 64 else 16)
        kblocks = -(-K // 64)
        assert -(-kblocks // parts) * (parts - 1) < kblocks       # no empty part
    assert ops.tile_plan(8, 32768, 2048, True, False) == (112, 1)       # 147 tiles for 148 SMs
