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
block table.  Which kernels do that is decided here, from the step context's facts
about the batch: 32-bit (and head sizes the tensor-core kernels are not built for)
runs the one-warp-per-row kernel, by row or by row and chunk of keys; bfloat16 sends
requests with one token to the split-key decode kernel and the others to the tiled
prefill kernel, which find their requests by q_len on the device.
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
                          self.position.rotary_dim, group.page_size, in_splits=parts,
                          pairing=getattr(self.position, "pairing", "half"))
        attn = ctx.buffer("attn", (n, self.nq * self.hd), self.model_dtype)
        self.attend(q, attn, k_pages, v_pages, ctx, cache.group)
        return as_branch(ops.project(attn, self.wo, lambda name, shape, dt: ctx.buffer("branch_" + name, shape, dt)))

    def attend(self, q, out, k_pages, v_pages, ctx, group: int) -> None:
        """Attention of every token of the step over its request's pages of cache group `group`."""
        nq, nkv, hd, window, scale = self.nq, self.nkv, self.hd, self.window or 0, self.scale
        ps, table = ctx.cache.page_size, ctx.group_tables[group]
        if q.dtype != torch.bfloat16 or not ops.mma_head_dim_ok(hd):
            # Three kernels with one result, bit for bit, so the choice is one of speed alone.  Portions of prompts:
            # 32 rows of a request share every tile of keys.  Few rows over long contexts (decoding): a warp per
            # (row, chunk of 64 keys).  Otherwise a warp per row.
            if ctx.num_multi > 0 and hd <= 256:
                ops.paged_attention_simt_tiled(q, out, k_pages, v_pages, ctx.req_q_start, ctx.req_q_len, ctx.req_ctx_len,
                                               table, ctx.max_q_len, nq, nkv, hd, ps, window, scale)
                return
            rows, chunks = q.shape[0] * nq, ops.simt_chunks(ctx.max_ctx, window)
            scratch = None
            if chunks > 1 and rows <= 4096 and rows * chunks <= 65536:
                scratch = ctx.buffer("attention_chunks", (rows * chunks * (hd + 2),), torch.float32)
            ops.paged_attention_simt(q, out, k_pages, v_pages, ctx.token_req, ctx.positions, table, nq, nkv, hd, ps,
                                     window, scale, scratch, chunks)
            return
        decode = ctx.num_single > 0 and nq // nkv <= 16
        if decode:
            R = ctx.n_requests
            # one CTA fits on an SM: every (request, kv head) is cut into parts so that the CTAs finish together
            # (planned for the context rounded up to 512 keys, so that a growing context seldom needs a new plan)
            split_keys, max_splits = ops.decode_split_plan(R * nkv, -(-ctx.max_ctx // 512) * 512, 32 if hd % 64 == 0 else 64)
            scratch = ctx.buffer("attention_splits", (ops.attention_mma_scratch_floats(R, nq, hd, max_splits),),
                                 torch.float32)
            ops.attention_mma_decode(q, out, k_pages, v_pages, ctx.req_q_start, ctx.req_q_len, ctx.req_ctx_len, table,
                                     nq, nkv, hd, ps, window, scale, split_keys, max_splits, scratch)
        if ctx.num_multi > 0 or not decode:
            split_above, halves = self._shared_tiles(ctx, skip_single=decode)
            ops.attention_mma_prefill(q, out, k_pages, v_pages, ctx.req_q_start, ctx.req_q_len, ctx.req_ctx_len, table,
                                      ctx.max_q_len, nq, nkv, hd, ps, window, scale, skip_single=decode,
                                      split_above=split_above, halves=halves)

    def _shared_tiles(self, ctx, skip_single: bool):
        """Whether this step's prefill attention shares its heavy tiles between two CTAs (ops.prefill_share_plan),
        and the buffer for their partial results.  Worked out once a step and head layout (kept in the step's
        memo), not once a layer; head sizes that run on pairs of CTAs (steps of 128, more than one tile of rows)
        never share."""
        nq, nkv, hd = self.nq, self.nkv, self.hd
        key = ("attention_share", nq, nkv, hd, skip_single)
        if key not in ctx.memo:
            if hd % 128 == 0 and ctx.max_q_len * (nq // nkv) > 128:
                plan = 0
            else:
                plan = ops.prefill_share_plan(ctx.host["req_q_len"].tolist(), ctx.host["req_ctx_len"].tolist(), nq, nkv,
                                              hd, skip_single)
            ctx.memo[key] = plan
        split_above = ctx.memo[key]
        if split_above <= 0:
            return 0, None
        floats = ops.attention_prefill_halves_floats(ctx.n_requests, ctx.max_q_len, nq, nkv, hd)
        return split_above, ctx.buffer("attention_halves", (floats,), torch.float32)
