"""Each part of a layer alone, built from a spec with sizes of its own, against the plain
function of tests/plain_gemma.py: norm, rotary table, attention mixer (fed in two portions
through a cache of its own), gated feed-forward, embedding and head, and a whole block."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_gemma as plain
from wllm_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, CacheRef, Residual, spec

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: dict(rtol=2e-5, atol=2e-5), torch.bfloat16: dict(rtol=3e-2, atol=3e-2)}


def whole(branch):
    """A branch output as one float32 tensor on the host (a step of few rows leaves it in partial sums)."""
    from wllm_b200.parts import Partials
    if isinstance(branch, Partials):
        return branch.tensor.float().sum(0).cpu()
    return branch.float().cpu()


def loader(tensors, dtype):
    return lambda name: tensors[name].to(DEV).to(dtype if tensors[name].dim() > 1 else tensors[name].dtype)


def runner_for(part_with_cache, dtype, page_size=16, pages=16, vocab=100, max_positions=4096):
    from wllm_b200.cache import CacheGroupSpec, CacheManager
    from wllm_b200.engine import ModelRunner
    need = part_with_cache.cache_need()
    groups = [CacheGroupSpec("g", 1, need.kv_heads, need.head_dim, need.window)]
    cache = CacheManager(groups, page_size, pages, 4, [], dtype, DEV)
    stub = SimpleNamespace(loaded=True, plan=SimpleNamespace(vocab_size=vocab, max_positions=max_positions))
    return ModelRunner(stub, cache, DEV)


def ctx_for(runner, rc, n):
    from wllm_b200.engine import StepEntry
    e = [StepEntry(rc, [0] * n, [])]
    runner.cache.reserve([(rc, n)])
    return runner._build(e)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,eps,unit", [(80, 1e-5, True), (1000, 1e-6, False)])
def test_norm_part(dtype, H, eps, unit):
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(H, generator=g) * 0.1).to(dtype)
    part = NORMS.build(spec("rmsnorm", weight="n.weight", eps=eps, unit_offset=unit), hidden_size=H, model_dtype=dtype)
    assert [(p.name, p.shape, p.kind) for p in part.param_specs()] == [("n.weight", (H,), "vector")]
    part.load(lambda name: w.to(DEV))
    x, branch = torch.randn(5, H, generator=g), torch.randn(5, H, generator=g).to(dtype)
    res = Residual(x.to(DEV))
    res.pending = branch.to(DEV)
    ctx = SimpleNamespace(buffer=lambda name, shape, dt: torch.empty(shape, dtype=dt, device=DEV))
    out = part(res, ctx)
    summed = x + branch.float()
    gain = w.float() if unit else w.float() - 1.0      # plain.rms_norm multiplies by (1 + w)
    assert res.pending is None and torch.equal(res.stream.cpu(), summed)
    torch.testing.assert_close(out.float().cpu(), plain.rms_norm(summed, gain, eps), **TOL[dtype])
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    torch.testing.assert_close(part.rows(res, rows, ctx).float().cpu(), plain.rms_norm(summed[[4, 1]], gain, eps), **TOL[dtype])


def test_rotary_table_follows_its_spec():
    p = POSITIONS.build(spec("rope", theta=500.0, head_dim=48))
    want = 1.0 / (500.0 ** (torch.arange(0, 48, 2, dtype=torch.float32) / 48))
    assert torch.equal(p.inv_freq, want) and p.rotary_dim == 48
    q = POSITIONS.build(spec("rope", theta=10000.0, head_dim=64, rotary_dim=32))
    assert q.inv_freq.shape == (16,) and q.rotary_dim == 32
    with pytest.raises(ValueError):
        POSITIONS.build(spec("rope", theta=1.0, head_dim=16, rotary_dim=18))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,nq,nkv,hd,theta", [(72, 6, 2, 16, 300.0), (64, 2, 2, 80, 10000.0), (96, 5, 1, 64, 50.0)])
def test_attention_mixer_in_two_portions(dtype, H, nq, nkv, hd, theta):
    g = torch.Generator().manual_seed(1)
    names = {k: f"a.{k}.weight" for k in ("q_proj", "k_proj", "v_proj", "o_proj")}
    part = MIXERS.build(spec("attention", num_heads=nq, num_kv_heads=nkv, head_dim=hd, window=None,
                             position=spec("rope", theta=theta, head_dim=hd), **names), hidden_size=H, model_dtype=dtype)
    tensors = {ps.name: (torch.randn(ps.shape, generator=g) * 0.08).to(torch.bfloat16).float() for ps in part.param_specs()}
    assert tensors[names["q_proj"]].shape == (nq * hd, H) and tensors[names["o_proj"]].shape == (H, nq * hd)
    part.load(loader(tensors, dtype))
    T, cut = 45, 29
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).float()
    cfg = dict(num_attention_heads=nq, num_key_value_heads=nkv, head_dim=hd, rope_theta=theta)
    w = {"p." + k.split(".", 1)[1]: v for k, v in tensors.items()}
    want = plain.self_attention(x, w, "p.", torch.arange(T), cfg)
    runner = runner_for(part, dtype)
    rc = runner.cache.open("r")
    outs = []
    for lo, hi in ((0, cut), (cut, T)):
        ctx = ctx_for(runner, rc, hi - lo)
        outs.append(whole(part(x[lo:hi].to(DEV).to(dtype), ctx, CacheRef(group=0, layer=0))).clone())
        runner.cache.commit(rc, hi - lo)
    torch.testing.assert_close(torch.cat(outs), want, **TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,I,act", [(72, 200, "gelu_tanh"), (64, 136, "silu")])
def test_gated_feed_forward_part(dtype, H, I, act):
    g = torch.Generator().manual_seed(2)
    names = {k: f"f.{k}.weight" for k in ("gate_proj", "up_proj", "down_proj")}
    part = FEED_FORWARDS.build(spec("gated_dense", intermediate_size=I, activation=act, **names), hidden_size=H, model_dtype=dtype)
    tensors = {ps.name: (torch.randn(ps.shape, generator=g) * 0.1).to(torch.bfloat16).float() for ps in part.param_specs()}
    part.load(loader(tensors, dtype))
    x = torch.randn(9, H, generator=g).to(torch.bfloat16).float()
    ctx = SimpleNamespace(buffer=lambda name, shape, dt: torch.empty(shape, dtype=dt, device=DEV))
    got = whole(part(x.to(DEV).to(dtype), ctx))
    wg, wu, wd = (tensors[names[k]] for k in ("gate_proj", "up_proj", "down_proj"))
    if act == "gelu_tanh":
        want = plain.feed_forward(x, wg, wu, wd)
    else:
        want = (torch.nn.functional.silu(x @ wg.T) * (x @ wu.T)) @ wd.T
    torch.testing.assert_close(got, want, **TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tied", [True, False])
def test_embedding_and_head(dtype, tied):
    from wllm_b200.parts.embedding import LogitsHead, ScaledEmbedding
    g = torch.Generator().manual_seed(3)
    V, H = 333, 96
    table = (torch.randn(V, H, generator=g) * 0.05).to(torch.bfloat16).float()
    head_w = (torch.randn(V, H, generator=g) * 0.05).to(torch.bfloat16).float()
    emb = ScaledEmbedding(spec("scaled_embedding", weight="e.weight", vocab_size=V, scale=math.sqrt(H),
                               scale_in_model_dtype=True), hidden_size=H, model_dtype=dtype)
    head = LogitsHead(spec("logits_head", tied=tied, weight="h.weight", vocab_size=V), hidden_size=H, model_dtype=dtype,
                      embedding=emb)
    assert [p.name for p in head.param_specs()] == ([] if tied else ["h.weight"])
    fetch = loader({"e.weight": table, "h.weight": head_w}, dtype)
    emb.load(fetch), head.load(fetch)
    ids = torch.randint(0, V, (7,), generator=g, dtype=torch.int32)
    ctx = SimpleNamespace(buffer=lambda name, shape, dt: torch.empty(shape, dtype=dt, device=DEV))
    x = emb(ids.to(DEV), ctx).cpu()
    factor = float(torch.tensor(math.sqrt(H)).to(dtype).float())       # the factor is held in the model's type
    assert x.dtype == torch.float32 and torch.equal(x, table[ids.long()] * factor)
    hidden = torch.randn(4, H, generator=g).to(torch.bfloat16).float()
    logits = head(hidden.to(DEV).to(dtype), ctx)
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits.cpu(), hidden @ (table if tied else head_w).T, **TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pre_norm_block(dtype):
    g = torch.Generator().manual_seed(4)
    H, I, nq, nkv, hd, eps, theta = 80, 176, 5, 5, 32, 1e-5, 777.0
    cfg = dict(hidden_size=H, intermediate_size=I, num_attention_heads=nq, num_key_value_heads=nkv, head_dim=hd,
               rms_norm_eps=eps, rope_theta=theta)
    p = "model.layers.0."
    block = BLOCKS.build(spec(
        "pre_norm", norm_in=spec("rmsnorm", weight=p + "input_layernorm.weight", eps=eps, unit_offset=True),
        mixer=spec("attention", num_heads=nq, num_kv_heads=nkv, head_dim=hd, window=None,
                   position=spec("rope", theta=theta, head_dim=hd), q_proj=p + "self_attn.q_proj.weight",
                   k_proj=p + "self_attn.k_proj.weight", v_proj=p + "self_attn.v_proj.weight",
                   o_proj=p + "self_attn.o_proj.weight"),
        norm_post=spec("rmsnorm", weight=p + "post_attention_layernorm.weight", eps=eps, unit_offset=True),
        feed_forward=spec("gated_dense", intermediate_size=I, activation="gelu_tanh", gate_proj=p + "mlp.gate_proj.weight",
                          up_proj=p + "mlp.up_proj.weight", down_proj=p + "mlp.down_proj.weight")),
        hidden_size=H, model_dtype=dtype)
    tensors = {}
    for part in block.parts():
        for ps in part.param_specs():
            tensors[ps.name] = (torch.randn(ps.shape, generator=g) * (0.1 if ps.kind == "vector" else 0.06)).to(torch.bfloat16).float()
        part.load(lambda name: tensors[name].to(DEV).to(dtype))
    T = 23
    x = torch.randn(T, H, generator=g)
    want = plain.decoder_layer(x, tensors, 0, torch.arange(T), cfg)
    runner = runner_for(block, dtype)
    rc = runner.cache.open("r")
    ctx = ctx_for(runner, rc, T)
    res = Residual(x.to(DEV).clone())
    block(res, ctx, CacheRef(group=0, layer=0))
    got = res.stream.cpu() + whole(res.pending)       # the last branch is still pending
    torch.testing.assert_close(got, want, **TOL[dtype])
