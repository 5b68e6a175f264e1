"""Configuration and registry: keys, defaults, and one error for all problems."""
import json

import pytest

from tiny_configs import TINY_A, TINY_B
from wllm_b200.config import ConfigError, EngineConfig, GemmaConfig, config_from_folder, resolve_architecture


def test_reads_every_size_from_its_own_keys():
    a, b = GemmaConfig.from_dict(TINY_A), GemmaConfig.from_dict(TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (2, 64, 4, 1, 32)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (3, 96, 3, 3, 48)
    assert (a.rope_theta, b.rope_theta, a.rms_norm_eps, b.rms_norm_eps) == (10000.0, 500.0, 1e-6, 1e-5)
    assert a.head_dim != a.hidden_size // a.num_attention_heads   # head size is its own key


def test_defaults_follow_the_reference_reader():
    raw = {"architectures": ["GemmaForCausalLM"], "vocab_size": 100, "hidden_size": 3072, "intermediate_size": 64,
           "num_hidden_layers": 1, "num_attention_heads": 16}
    c = GemmaConfig.from_dict(raw)
    assert c.num_key_value_heads == 16 and c.head_dim == 192 and c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0
    assert c.max_position_embeddings == 4096 and c.tie_word_embeddings is True and c.attention_bias is False
    assert GemmaConfig.from_dict(dict(raw, head_dim=256)).head_dim == 256
    assert GemmaConfig.from_dict(dict(raw, rope_parameters={"rope_theta": 777.0})).rope_theta == 777.0
    assert GemmaConfig.from_dict(dict(raw, eos_token_id=[1, 107])).eos_token_id == 1


def test_all_problems_in_one_error():
    raw = dict(TINY_A)
    del raw["vocab_size"], raw["intermediate_size"]
    raw["num_hidden_layers"] = "two"
    raw["hidden_act"] = "relu"
    with pytest.raises(ConfigError) as e:
        GemmaConfig.from_dict(raw)
    msg = str(e.value)
    for piece in ("vocab_size", "intermediate_size", "num_hidden_layers", "relu"):
        assert piece in msg


@pytest.mark.parametrize("change,word", [({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 31}, "odd"),
                                          ({"attention_bias": True}, "bias"), ({"rope_scaling": {"type": "linear"}}, "rope_scaling"),
                                          ({"hidden_size": -4}, "hidden_size"), ({"rope_theta": 0}, "rope_theta")])
def test_refuses_what_it_cannot_run(change, word):
    with pytest.raises(ConfigError, match=word):
        GemmaConfig.from_dict(dict(TINY_A, **change))


def test_registry_resolves_and_names_what_it_knows(tmp_path):
    assert resolve_architecture(["Nope", "GemmaForCausalLM"]).config_class is GemmaConfig
    with pytest.raises(ConfigError, match="GemmaForCausalLM"):
        resolve_architecture(["LlamaForCausalLM"])
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    arch, cfg = config_from_folder(str(tmp_path))
    assert arch.name == "GemmaForCausalLM" and cfg.vocab_size == 1000
    plan = arch.make_plan(cfg)
    assert len(plan.blocks) == 3 and plan.blocks[0].mixer.head_dim == 48 and plan.blocks[2].norm_in.eps == 1e-5
    with pytest.raises(ConfigError, match="no such file"):
        config_from_folder(str(tmp_path / "missing"))


def test_round_trip_through_to_dict():
    c = GemmaConfig.from_dict(TINY_B)
    assert GemmaConfig.from_dict(c.to_dict()) == c


def test_engine_config_checks():
    assert EngineConfig(dtype="float32").dtype.is_floating_point
    for bad in (dict(block_size=24), dict(block_size=8), dict(num_blocks=0), dict(dtype="float16"),
                dict(chunked_prefill_tokens=0), dict(prefill_row_quantum=-1)):
        with pytest.raises(ConfigError):
            EngineConfig(**bad)
    # the scheduler's tile of rows follows the element type unless it is given
    assert EngineConfig(dtype="bfloat16").prefill_row_quantum == 256
    assert EngineConfig(dtype="float32").prefill_row_quantum == 0
    assert EngineConfig(dtype="bfloat16", prefill_row_quantum=0).prefill_row_quantum == 0
