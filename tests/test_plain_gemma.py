"""The plain implementation against the outputs of the reference's own model class, made
once by tests/golden/make_golden.py, and its parts against hand-computed values."""
import math
import os

import pytest
import torch
from safetensors.torch import load_file

import plain_gemma as plain
from tiny_configs import CONFIGS, SEEDS

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B"])
def test_matches_the_reference_models_logits_and_greedy_tokens(name):
    gold = load_file(os.path.join(GOLDEN, f"golden_{name}.safetensors"))
    w = plain.random_weights(CONFIGS[name], SEEDS[name])
    logits = plain.forward(gold["ids"], w, CONFIGS[name])
    assert float((logits - gold["logits"]).abs().max()) < 2e-6
    assert torch.equal(logits.argmax(-1), gold["logits"].argmax(-1))
    assert plain.greedy(gold["prompt"].tolist(), w, CONFIGS[name], 16) == gold["greedy"].tolist()


def test_norm_gain_is_one_plus_weight():
    x = torch.tensor([[3.0, 4.0]])
    out = plain.rms_norm(x, torch.tensor([0.0, 1.0]), 0.0)
    rms = math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[3.0 / rms, 8.0 / rms]]))


def test_rotary_pairs_and_frequencies():
    cos, sin = plain.rope_tables(torch.tensor([0, 3]), 4, 100.0)
    assert torch.allclose(cos[0], torch.ones(4)) and torch.allclose(sin[0], torch.zeros(4))
    assert torch.allclose(sin[1], torch.tensor([math.sin(3.0), math.sin(0.3), math.sin(3.0), math.sin(0.3)]), atol=1e-6)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]])
    assert torch.equal(plain.rotate_half(x), torch.tensor([[[-3.0, -4.0, 1.0, 2.0]]]))


def test_gelu_is_the_tanh_approximation():
    x = torch.tensor([-2.0, 0.0, 1.5])
    assert torch.allclose(plain.gelu_tanh(x), torch.nn.functional.gelu(x, approximate="tanh"), atol=1e-7)
    assert not torch.allclose(plain.gelu_tanh(x), torch.nn.functional.gelu(x), atol=1e-5)


def test_attention_is_causal_grouped_and_scaled():
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(5, 4, 8, generator=g), torch.randn(5, 2, 8, generator=g), torch.randn(5, 2, 8, generator=g)
    out = plain.attention(q, k, v)
    assert torch.allclose(out[0, 3], v[0, 1])                      # first token sees itself only; head 3 -> group 1
    s = (q[2, 1] @ k[:3, 0].T) / math.sqrt(8)
    assert torch.allclose(out[2, 1], torch.softmax(s, 0) @ v[:3, 0], atol=1e-6)
    win = plain.attention(q, k, v, window=2)
    s2 = (q[4, 0] @ k[3:5, 0].T) / math.sqrt(8)
    assert torch.allclose(win[4, 0], torch.softmax(s2, 0) @ v[3:5, 0], atol=1e-6)


def test_embedding_scaled_head_not():
    cfg = dict(CONFIGS["A"])
    w = plain.random_weights(cfg, 1)
    assert torch.allclose(plain.embed(torch.tensor([5]), w["model.embed_tokens.weight"], 64),
                          w["model.embed_tokens.weight"][5:6] * 8.0)
    h = torch.randn(2, 64)
    assert torch.equal(plain.logits_head(h, w, cfg), h @ w["model.embed_tokens.weight"].T)


def test_sampling_filters_follow_the_reference_rules():
    logits = torch.log(torch.tensor([0.5, 0.25, 0.15, 0.1]))
    assert plain.kept_mask(logits, 2, 1.0, 0.0).tolist() == [True, True, False, False]
    assert plain.kept_mask(logits, 0, 0.8, 0.0).tolist() == [True, True, False, False]   # cumsum 0.5, 0.75 <= 0.8 < 0.9
    assert plain.kept_mask(logits, 0, 0.3, 0.0).tolist() == [True, False, False, False]  # rank 0 always stays
    assert plain.kept_mask(logits, 0, 1.0, 0.4).tolist() == [True, True, False, False]   # p >= 0.4 * 0.5
    pen = plain.penalise_repeats(torch.tensor([2.0, -2.0, 1.0]), [0, 1, 1], 2.0)
    assert pen.tolist() == [1.0, -4.0, 1.0]
    probs, logp = plain.sampling_distribution(torch.tensor([1.0, 3.0, 2.0]), 0.0)
    assert probs.tolist() == [0.0, 1.0, 0.0] and abs(float(logp.exp().sum()) - 1) < 1e-9
