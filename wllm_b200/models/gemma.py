"""Gemma 1 as a plan of parts.

Every layer is a pre-norm block of (1+w) RMSNorm, rotary attention over all keys,
(1+w) RMSNorm and a tanh-GELU gated feed-forward; the embedding is scaled by
sqrt(hidden_size) and the head is tied to it (src/wllm/models/gemma.py:41-173).
Tensor names are the checkpoint's (src/wllm/models/llama.py:1-4).
"""
from __future__ import annotations

from ..config.gemma import GemmaConfig
from ..config.registry import register_architecture
from ..parts import ModelPlan, spec


@register_architecture("GemmaForCausalLM", GemmaConfig)
def gemma_plan(cfg: GemmaConfig) -> ModelPlan:
    blocks = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        blocks.append(spec(
            "pre_norm",
            norm_in=spec("rmsnorm", weight=p + "input_layernorm.weight", eps=cfg.rms_norm_eps, unit_offset=True),
            mixer=spec("attention", num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
                       head_dim=cfg.head_dim, window=None,
                       position=spec("rope", theta=cfg.rope_theta, head_dim=cfg.head_dim),
                       q_proj=p + "self_attn.q_proj.weight", k_proj=p + "self_attn.k_proj.weight",
                       v_proj=p + "self_attn.v_proj.weight", o_proj=p + "self_attn.o_proj.weight"),
            norm_post=spec("rmsnorm", weight=p + "post_attention_layernorm.weight", eps=cfg.rms_norm_eps,
                           unit_offset=True),
            feed_forward=spec("gated_dense", intermediate_size=cfg.intermediate_size, activation="gelu_tanh",
                              gate_proj=p + "mlp.gate_proj.weight", up_proj=p + "mlp.up_proj.weight",
                              down_proj=p + "mlp.down_proj.weight"),
        ))
    return ModelPlan(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
        embedding=spec("scaled_embedding", weight="model.embed_tokens.weight", vocab_size=cfg.vocab_size,
                       scale=float(cfg.hidden_size) ** 0.5, scale_in_model_dtype=True),
        blocks=blocks,
        final_norm=spec("rmsnorm", weight="model.norm.weight", eps=cfg.rms_norm_eps, unit_offset=True),
        head=spec("logits_head", tied=cfg.tie_word_embeddings, weight="lm_head.weight", vocab_size=cfg.vocab_size),
        eos_token_id=cfg.eos_token_id, bos_token_id=cfg.bos_token_id,
    )
