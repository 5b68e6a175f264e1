"""Gemma 1 (`GemmaForCausalLM`) configuration, read from its own config.json keys.

Keys and defaults follow the reference's reader (src/wllm/models/config.py:38-71):
`num_key_value_heads` defaults to the number of query heads, `head_dim` to
hidden_size // num_attention_heads, `rms_norm_eps` to 1e-6, `rope_theta` to 10000
(also read from `rope_parameters.rope_theta`), `max_position_embeddings` to 4096.
Two defaults differ on purpose: `tie_word_embeddings` is true when absent (a Gemma
checkpoint has no lm_head tensor), and `attention_bias` is false.  The activation
is the tanh approximation of GELU (src/wllm/models/gemma.py:62); a config.json
that names another one is refused instead of silently run with the wrong function.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass

from .base import ConfigError, ConfigReader

_TANH_GELU_NAMES = ("gelu_pytorch_tanh", "gelu_tanh", "gelu_new", "gelu")


@dataclass(frozen=True)
class GemmaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 4096
    tie_word_embeddings: bool = True
    attention_bias: bool = False
    eos_token_id: int | None = None
    bos_token_id: int | None = None

    architecture = "GemmaForCausalLM"

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "GemmaConfig":
        r = ConfigReader(raw, where)
        heads = r.integer("num_attention_heads")
        hidden = r.integer("hidden_size")
        rope_theta = raw.get("rope_theta")
        if rope_theta is None and isinstance(raw.get("rope_parameters"), dict):
            rope_theta = raw["rope_parameters"].get("rope_theta")
        if rope_theta is not None and (isinstance(rope_theta, bool) or not isinstance(rope_theta, (int, float)) or rope_theta <= 0):
            r.complain(f"'rope_theta' must be a positive number, got {rope_theta!r}")
            rope_theta = None
        eos = raw.get("eos_token_id")
        if isinstance(eos, list):  # some checkpoints list several; the first one ends a request
            eos = eos[0] if eos else None
        cfg = cls(
            vocab_size=r.integer("vocab_size"),
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size"),
            num_hidden_layers=r.integer("num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=r.integer("num_key_value_heads", default=heads),
            head_dim=r.integer("head_dim", default=(hidden // heads if hidden and heads else None)),
            rms_norm_eps=r.number("rms_norm_eps", default=1e-6),
            rope_theta=float(rope_theta) if rope_theta is not None else 10000.0,
            max_position_embeddings=r.integer("max_position_embeddings", default=4096),
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=True),
            attention_bias=r.boolean("attention_bias", default=False),
            eos_token_id=eos if isinstance(eos, int) else None,
            bos_token_id=raw.get("bos_token_id") if isinstance(raw.get("bos_token_id"), int) else None,
        )
        for key in ("hidden_act", "hidden_activation"):
            act = raw.get(key)
            if act is not None and act not in _TANH_GELU_NAMES:
                r.complain(f"'{key}' = {act!r}: Gemma 1 runs tanh-approximated GELU only ({', '.join(_TANH_GELU_NAMES)})")
        if raw.get("rope_scaling") is not None:
            r.complain("'rope_scaling' is set: scaled rotary frequencies are not part of Gemma 1")
        r.finish()
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "GemmaConfig") -> None:
        problems = []
        if self.num_attention_heads % self.num_key_value_heads:
            problems.append(f"num_attention_heads {self.num_attention_heads} is no multiple of "
                            f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            problems.append(f"head_dim {self.head_dim} is odd: rotary pairs need an even size")
        if self.attention_bias:
            problems.append("attention_bias is true: Gemma 1 projections have no bias")
        if problems:
            raise ConfigError(f"{where}: " + "; ".join(problems))

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = "gemma"
        d["hidden_act"] = "gelu_pytorch_tanh"
        return d
