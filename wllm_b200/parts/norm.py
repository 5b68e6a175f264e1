"""Root-mean-square norm with the residual add folded in.

spec options: weight (checkpoint name), eps, unit_offset (True: gain is 1 + w, as
Gemma stores it, src/wllm/models/gemma.py:42-51; False: gain is w).
The statistics and the gain are applied in 32-bit on the 32-bit residual; the
result is rounded once to the model's element type.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import NORMS, ParamSpec, Residual


@NORMS.register("rmsnorm")
class RMSNorm:
    graph_safe = True
    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.weight_name = spec.weight
        self.eps = float(spec.eps)
        self.offset = 1.0 if spec.unit_offset else 0.0
        self.hidden_size = hidden_size
        self.model_dtype = model_dtype
        self.weight = None

    def param_specs(self):
        return [ParamSpec(self.weight_name, (self.hidden_size,), "vector")]

    def load(self, fetch):
        self.weight = fetch(self.weight_name)

    def __call__(self, residual: Residual, ctx) -> torch.Tensor:
        out = ctx.buffer("normed", (residual.stream.shape[0], self.hidden_size), self.model_dtype)
        delta, parts = residual.pending_args()
        ops.rmsnorm(residual.stream, delta, self.weight, self.eps, self.offset, out, delta_splits=parts)
        residual.pending = None
        return out

    def rows(self, residual: Residual, rows: torch.Tensor, ctx) -> torch.Tensor:
        out = torch.empty((rows.shape[0], self.hidden_size), dtype=self.model_dtype, device=rows.device)
        delta, parts = residual.pending_args()
        ops.rmsnorm(residual.stream, delta, self.weight, self.eps, self.offset, out, rows=rows, delta_splits=parts)
        return out
