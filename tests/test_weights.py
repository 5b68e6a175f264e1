"""Weights by tensor name: element types, one error for all mismatches, random-weights folders."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from tiny_configs import TINY_A, TINY_B
from wllm_b200.config import config_from_folder
from wllm_b200.engine import ComposedModel
from wllm_b200.weights import WeightError, load_weights, random_tensors, write_random_model


def model_of(folder, dtype):
    arch, cfg = config_from_folder(folder)
    return ComposedModel(arch.make_plan(cfg), dtype)


def test_random_folder_is_reproducible_and_complete(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_A, 7)
    b = write_random_model(str(tmp_path / "b"), TINY_A, 7)
    c = write_random_model(str(tmp_path / "c"), TINY_A, 8)
    ta, tb, tc = (load_file(os.path.join(f, "model.safetensors")) for f in (a, b, c))
    assert set(ta) == set(tb) and all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["model.embed_tokens.weight"], tc["model.embed_tokens.weight"])
    assert "lm_head.weight" not in ta and len(ta) == 2 + 9 * TINY_A["num_hidden_layers"]
    assert ta["model.layers.1.self_attn.q_proj.weight"].shape == (4 * 32, 64)
    assert ta["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert abs(float(ta["model.embed_tokens.weight"].float().std()) - 0.02) < 0.002
    assert abs(float(ta["model.norm.weight"].float().std()) - 0.1) < 0.03
    assert json.load(open(os.path.join(a, "config.json")))["architectures"] == ["GemmaForCausalLM"]


def test_loads_by_name_and_fuses(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_B, 3)
    raw = load_file(os.path.join(folder, "model.safetensors"))
    for dtype in (torch.bfloat16, torch.float32):
        m = model_of(folder, dtype)
        load_weights(m, folder, "cpu")
        att = m.blocks[1].mixer
        want = torch.cat([raw[f"model.layers.1.self_attn.{n}_proj.weight"] for n in "qkv"]).to(dtype)
        assert att.wqkv.dtype == dtype and torch.equal(att.wqkv, want)
        assert m.blocks[2].feed_forward.wgu.shape == (2 * 384, 96)
        assert m.head.weight is m.embedding.table          # tied: one tensor, read once
        assert m.final_norm.weight.dtype == dtype


def test_a_tensor_stored_in_32bit_stays_so(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, 3)
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    t["model.norm.weight"] = t["model.norm.weight"].float() + 1e-4   # not representable in bfloat16
    save_file(t, path)
    m = model_of(folder, torch.bfloat16)
    load_weights(m, folder, "cpu")
    assert m.final_norm.weight.dtype == torch.float32 and torch.equal(m.final_norm.weight, t["model.norm.weight"])
    assert m.blocks[0].norm_in.weight.dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, 3)
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    del t["model.layers.0.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.9.extra.weight"] = torch.zeros(2)
    t["lm_head.weight"] = torch.zeros(512, 64)
    t["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(64, 64)
    save_file(t, path)
    with pytest.raises(WeightError) as e:
        load_weights(model_of(folder, torch.bfloat16), folder, "cpu")
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.0.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected tensors (2)" in msg and "model.layers.9.extra.weight" in msg and "lm_head.weight" in msg
    assert "wrong shapes (1)" in msg and "expected (32, 64), file has (64, 64)" in msg


def test_untied_head_has_its_own_tensor(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), dict(TINY_A, tie_word_embeddings=False), 3)
    assert "lm_head.weight" in load_file(os.path.join(folder, "model.safetensors"))
    m = model_of(folder, torch.float32)
    load_weights(m, folder, "cpu")
    assert m.head.weight is not m.embedding.table


def test_no_safetensors_is_said_plainly(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(WeightError, match="no .safetensors"):
        load_weights(model_of(str(tmp_path), torch.float32), str(tmp_path), "cpu")


def test_random_tensors_names_follow_the_plan():
    names = set(random_tensors(TINY_B, 1))
    assert "model.layers.2.post_attention_layernorm.weight" in names and len(names) == 2 + 9 * 3
