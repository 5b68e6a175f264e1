"""Gated dense feed-forward: down(act(gate(x)) * up(x)).

spec options: intermediate_size, activation ('gelu_tanh' for Gemma's GeGLU,
src/wllm/models/gemma.py:54-62; 'silu'), gate_proj/up_proj/down_proj (checkpoint
names).  gate and up are stored as one matrix [2 I, hidden] (gate rows first).  Under
bfloat16 one tensor-memory GEMM computes both products and applies act(gate) * up in its
epilogue, in 32-bit on the accumulators; otherwise one product feeds the activation kernel.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FEED_FORWARDS, ParamSpec, as_branch


@FEED_FORWARDS.register("gated_dense")
class GatedDense:
    graph_safe = True
    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.inter = int(spec.intermediate_size)
        self.activation = spec.activation
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.names = {k: spec.options[k] for k in ("gate_proj", "up_proj", "down_proj")}
        self.wgu = self.wd = None

    def param_specs(self):
        H, I, n = self.hidden_size, self.inter, self.names
        return [ParamSpec(n["gate_proj"], (I, H)), ParamSpec(n["up_proj"], (I, H)), ParamSpec(n["down_proj"], (H, I))]

    def load(self, fetch):
        n = self.names
        self.wgu = torch.cat([fetch(n["gate_proj"]), fetch(n["up_proj"])], dim=0).contiguous()
        self.wd = fetch(n["down_proj"]).contiguous()

    def __call__(self, x: torch.Tensor, ctx):
        n = x.shape[0]
        h = ops.gated_linear(x, self.wgu, self.activation, ctx.buffer("ffn_act", (n, self.inter), self.model_dtype),
                             lambda shape, dtype: ctx.buffer("gate_up", shape, dtype))
        return as_branch(ops.project(h, self.wd, lambda name, shape, dt: ctx.buffer("branch_" + name, shape, dt)))
