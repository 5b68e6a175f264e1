"""The two tiny Gemma 1 configurations of the tests, as config.json dictionaries.

They differ in every size and option: layers, width, query heads and groups
(MQA against MHA), head size (neither equals width/heads), feed-forward width,
vocabulary (one no power of two), rope base, the norms' eps, and the page size
the tests pair them with.  Gemma 1 has no window, experts or scale factors.
"""

TINY_A = {
    "architectures": ["GemmaForCausalLM"],
    "model_type": "gemma",
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 1,
    "head_dim": 32,
    "intermediate_size": 256,
    "vocab_size": 512,
    "max_position_embeddings": 256,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "hidden_act": "gelu_pytorch_tanh",
    "tie_word_embeddings": True,
    "attention_bias": False,
    "bos_token_id": 2,
    "eos_token_id": 1,
}

TINY_B = {
    "architectures": ["GemmaForCausalLM"],
    "model_type": "gemma",
    "num_hidden_layers": 3,
    "hidden_size": 96,
    "num_attention_heads": 3,
    "num_key_value_heads": 3,
    "head_dim": 48,
    "intermediate_size": 384,
    "vocab_size": 1000,
    "max_position_embeddings": 512,
    "rope_theta": 500.0,
    "rms_norm_eps": 1e-5,
    "hidden_activation": "gelu_pytorch_tanh",
    "tie_word_embeddings": True,
    "attention_bias": False,
    "bos_token_id": 2,
    "eos_token_id": 1,
}

# seed of the random weights and page size that the tests pair with each
SEEDS = {"A": 11, "B": 23}
PAGE_SIZES = {"A": 16, "B": 32}
CONFIGS = {"A": TINY_A, "B": TINY_B}
