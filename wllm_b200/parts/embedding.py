"""Token embedding (scaled) and the logits head (tied to it or with a matrix of its own).

Embedding spec options: weight (checkpoint name), vocab_size, scale, and
scale_in_model_dtype: Gemma multiplies by sqrt(hidden_size) held in the model's
element type (src/wllm/models/llama.py:397-403, src/wllm/models/gemma.py:158-162),
so under bfloat16 the factor is the bfloat16 value nearest to the square root; the
product itself goes to the 32-bit residual unrounded.
Head spec options: tied (bool), weight (checkpoint name when not tied), vocab_size.
The tied head multiplies by the unscaled table (src/wllm/models/llama.py:443-446) and
is evaluated only at the rows whose logits are wanted; logits are 32-bit.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import EMBEDDINGS, HEADS, ParamSpec


@EMBEDDINGS.register("scaled_embedding")
class ScaledEmbedding:
    graph_safe = True
    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.weight_name, self.vocab = spec.weight, int(spec.vocab_size)
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        scale = float(spec.options.get("scale", 1.0))
        if spec.options.get("scale_in_model_dtype", False):
            scale = float(torch.tensor(scale, dtype=torch.float32).to(model_dtype).to(torch.float32))
        else:
            scale = float(torch.tensor(scale, dtype=torch.float32))
        self.scale = scale
        self.table = None

    def param_specs(self):
        return [ParamSpec(self.weight_name, (self.vocab, self.hidden_size), "table")]

    def load(self, fetch):
        self.table = fetch(self.weight_name).contiguous()

    def __call__(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        out = ctx.buffer("residual", (token_ids.shape[0], self.hidden_size), torch.float32)
        return ops.embed_gather(token_ids, self.table, self.scale, out)


@HEADS.register("logits_head")
class LogitsHead:
    graph_safe = True
    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype, embedding: ScaledEmbedding):
        self.tied = bool(spec.tied)
        self.vocab = int(spec.vocab_size)
        self.weight_name = None if self.tied else spec.weight
        self.hidden_size, self.model_dtype, self.embedding = hidden_size, model_dtype, embedding
        self.weight = None

    def param_specs(self):
        return [] if self.tied else [ParamSpec(self.weight_name, (self.vocab, self.hidden_size), "table")]

    def load(self, fetch):
        self.weight = self.embedding.table if self.tied else fetch(self.weight_name).contiguous()

    def __call__(self, hidden_rows: torch.Tensor, ctx) -> torch.Tensor:
        if self.weight is None:
            self.weight = self.embedding.table
        return ops.linear(hidden_rows, self.weight, f32_out=True)
