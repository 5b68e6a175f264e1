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


@pytest.mark.parametrize("M,N,K", [(8, 2048, 2048), (8, 2560, 2048), (64, 2048, 16384), (1, 512, 200), (33, 300, 1024)])
def test_split_k_partial_sums(M, N, K):
    from wllm_b200.kernels import ops
    a, w = operands(M, N, K, seed=K + M)
    want = a.double() @ w.double().T
    parts = ops.split_plan(M, N, K)
    assert parts >= 1 and (K <= 64 or parts > 1)
    out = torch.full((parts, M, N), float("nan"), device=DEV)
    if parts > 1:
        ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), out=out, epilogue="f32", k_splits=parts)
    else:
        ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), out=out[0], epilogue="f32")
    torch.cuda.synchronize()
    assert ops.tc_gemm_status(DEV) == 0
    total = out.cpu().double().sum(0)
    torch.testing.assert_close(total, want, rtol=1e-4, atol=1e-3 * math.sqrt(K))
    again = torch.empty_like(out)
    ops.gemm_bf16_tc(a.to(DEV), w.to(DEV), out=again if parts > 1 else again[0], epilogue="f32", k_splits=parts)
    assert torch.equal(again, out)        # part s is the same sum whoever computes it
