"""Attention over the paged cache: fused q|k|v projection, rotary encoding and cache
write, attention, output projection.

spec options: num_heads, num_kv_heads, head_dim, position (a position spec),
window (None or a number of keys), q_proj/k_proj/v_proj/o_proj (checkpoint names).
Query head h reads key/value head h // (num_heads/num_kv_heads); scores are scaled
by head_dim^-0.5 (src/wllm/models/llama.py:74-79, 242).  The three projections are
stored as one matrix [(nq + 2 nkv) * hd, hidden], rows in the order q, k, v, so one
product replaces three (the reference runs three, src/wllm/models/llama.py:103-105).

One forward serves whole prompts, portions and decoded tokens alike: the step's keys
and values go into the pages first, then every token attends through its request's
block table.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, POSITIONS, CacheRef, KVNeed, ParamSpec, as_branch


@MIXERS.register("attention")
class PagedAttention:
    graph_safe = True
    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.nq, self.nkv, self.hd = int(spec.num_heads), int(spec.num_kv_heads), int(spec.head_dim)
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads are no multiple of {self.nkv} key/value heads")
        if self.hd % 16:
            raise ValueError(f"head_dim {self.hd}: the attention kernels take head sizes in steps of 16")
        self.window = spec.options.get("window")
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.names = {k: spec.options[k] for k in ("q_proj", "k_proj", "v_proj", "o_proj")}
        self.position = POSITIONS.build(spec.position)
        self.scale = float(self.hd) ** -0.5
        self.wqkv = self.wo = None

    def cache_need(self):
        return KVNeed(self.nkv, self.hd, self.window)

    def param_specs(self):
        H, n = self.hidden_size, self.names
        return [ParamSpec(n["q_proj"], (self.nq * self.hd, H)), ParamSpec(n["k_proj"], (self.nkv * self.hd, H)),
                ParamSpec(n["v_proj"], (self.nkv * self.hd, H)), ParamSpec(n["o_proj"], (H, self.nq * self.hd))]

    def load(self, fetch):
        n = self.names
        self.wqkv = torch.cat([fetch(n["q_proj"]), fetch(n["k_proj"]), fetch(n["v_proj"])], dim=0).contiguous()
        self.wo = fetch(n["o_proj"]).contiguous()
        self.position.to(self.wo.device)

    def __call__(self, x: torch.Tensor, ctx, cache: CacheRef):
        n = x.shape[0]
        qkv, parts = ops.project(x, self.wqkv, lambda name, shape, dt: ctx.buffer("qkv_" + name, shape, dt))
        group = ctx.cache.groups[cache.group]
        k_pages, v_pages = group.keys(cache.layer), group.values(cache.layer)
        q = ctx.buffer("q_rotated", (n, self.nq * self.hd), self.model_dtype)
        ops.rope_kv_write(qkv, q, ctx.positions, ctx.group_slots[cache.group] if cache.writes else None,
                          self.position.inv_freq, k_pages, v_pages, self.nq, self.nkv, self.hd,
                          self.position.rotary_dim, group.page_size, in_splits=parts)
        attn = ctx.buffer("attn", (n, self.nq * self.hd), self.model_dtype)
        ctx.attention(q, attn, k_pages, v_pages, cache.group, self.nq, self.nkv, self.hd, self.window or 0, self.scale)
        return as_branch(ops.project(attn, self.wo, lambda name, shape, dt: ctx.buffer("branch_" + name, shape, dt)))
